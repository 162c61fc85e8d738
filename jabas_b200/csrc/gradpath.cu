// Gradient-path kernels for B200 (sm_100a) and their C ABI (include/jabas_b200.h).
//
// Everything here is HBM-bound streaming work: no tensor cores, no shared-memory
// tiling beyond the reduction trees.  Design points:
//   * 128-bit loads/stores, block-cyclic tiles so that a warp always touches 512
//     contiguous bytes per stream, all loads of a tile issued before the first use;
//   * grids of (SM count x resident CTAs) persistent CTAs walking the buffer;
//   * fp32 arithmetic written with explicit-rounding intrinsics (__fmaf_rn, __fmul_rn,
//     __fadd_rn, __fdiv_rn, __fsqrt_rn) so that the result is bit-identical to the CPU
//     oracle whatever the compiler's contraction rules are;
//   * the three sums of the cosine statistic accumulate in fp64 per thread, reduce by
//     warp shuffle and a shared-memory tree to one partial per CTA, and the last CTA
//     to finish (ticket counter) adds the partials in index order: the result does
//     not depend on scheduling.
#include "common.cuh"

#include <cstdio>
#include <new>
#include <vector>

namespace {
thread_local std::string g_err;
}

int jb_fail(int code, const std::string& msg)
{
    g_err = msg;
    return code;
}

namespace {

// ---- bulk-copy (TMA, untiled) staging of tiles into shared memory ------------------------
// One elected thread issues `cp.async.bulk` for every input stream of a tile; the copies
// complete on an mbarrier of the stage, which the CTA's threads poll with a bounded number
// of `try_wait`s.  Source, destination and byte count are multiples of 16 by construction
// (16-byte aligned buffers, tiles of 4 KB, tails in whole 4-vectors).
constexpr int kMaxStages = 4;
constexpr int kStageTileVecs = kThreads;                 // one 4-vector per thread and stream
constexpr unsigned kStageTileBytes = kStageTileVecs * 16; // 4 KB per stream and stage
constexpr int kStageBudgetBytes = 72 * 1024;             // dynamic shared memory asked per CTA


// One partial per CTA; the last CTA to arrive adds them in CTA order into stat3.
__device__ __forceinline__ void stat_finish(Acc3 acc, StatWs ws, double* stat3)
{
    __shared__ double sm[3][kWarps];
    __shared__ int is_last;
    Acc3 r = block_sum(acc, sm);
    if (threadIdx.x == 0) {
        ws.partials[3 * blockIdx.x + 0] = r.d;
        ws.partials[3 * blockIdx.x + 1] = r.a;
        ws.partials[3 * blockIdx.x + 2] = r.b;
        __threadfence();
        const unsigned int t = atomicAdd(ws.counter, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Acc3 t = {0.0, 0.0, 0.0};
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += kThreads) {
        t.d += __ldcg(ws.partials + 3 * i + 0);
        t.a += __ldcg(ws.partials + 3 * i + 1);
        t.b += __ldcg(ws.partials + 3 * i + 2);
    }
    t = block_sum(t, sm);
    if (threadIdx.x == 0) {
        stat3[0] += t.d; stat3[1] += t.a; stat3[2] += t.b;
        *ws.counter = 0u;
    }
}

// ----------------------------------------------------------------------------------
// K-VSW aggregation
// ----------------------------------------------------------------------------------

struct AggArgs {
    const float* g[JABAS_MAX_VSW];
    float* out;
    float* half;     // nullable
    double* stat;    // nullable (STAT kernels only)
    StatWs ws;
    unsigned long long n;
    float divisor;
    float half_divisor;
    int K;
};

__host__ __device__ constexpr int agg_unroll(int K) { return K <= 2 ? 4 : (K <= 4 ? 2 : 1); }

// Per-element form: the tail of the vector kernel and the whole of the unaligned path.
template <bool STAT>
__device__ __forceinline__ void agg_elem(const AggArgs& a, unsigned long long i, Acc3& acc)
{
    float s = a.g[0][i];
    float e = s, o = 0.0f;
    for (int k = 1; k < a.K; ++k) {
        const float x = a.g[k][i];
        s = __fadd_rn(s, x);
        if (STAT) {
            if (k == 1) o = x;
            else if (k & 1) o = __fadd_rn(o, x);
            else e = __fadd_rn(e, x);
        }
    }
    if (a.half) a.half[i] = s;
    a.out[i] = __fdiv_rn(s, a.divisor);
    if (STAT) acc_one(acc, __fdiv_rn(e, a.half_divisor), __fdiv_rn(o, a.half_divisor));
}

template <int K, bool STAT>
__global__ void __launch_bounds__(kThreads) agg_vec_kernel(const AggArgs a)
{
    constexpr int U = agg_unroll(K);
    const unsigned long long nvec = a.n >> 2;
    const unsigned long long tile = (unsigned long long)kThreads * U;
    Acc3 acc = {0.0, 0.0, 0.0};
    for (unsigned long long t0 = (unsigned long long)blockIdx.x * tile; t0 < nvec;
         t0 += (unsigned long long)gridDim.x * tile) {
        float4 x[U][K];
        const bool full = t0 + tile <= nvec;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
            if (full || v < nvec) {
#pragma unroll
                for (int k = 0; k < K; ++k) x[u][k] = ld4(a.g[k] + 4 * v);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
            if (full || v < nvec) {
                float4 s = x[u][0];
#pragma unroll
                for (int k = 1; k < K; ++k) s = add4(s, x[u][k]);
                if (a.half) st4(a.half + 4 * v, s);
                st4(a.out + 4 * v, div4(s, a.divisor));
                if (STAT) {
                    float4 e = x[u][0];
                    float4 o = K > 1 ? x[u][K > 1 ? 1 : 0] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int k = 2; k < K; ++k) {
                        if (k & 1) o = add4(o, x[u][k]); else e = add4(e, x[u][k]);
                    }
                    acc_vec(acc, div4(e, a.half_divisor), div4(o, a.half_divisor));
                }
            }
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < (a.n & 3ull))
        agg_elem<STAT>(a, (nvec << 2) + threadIdx.x, acc);
    if (STAT) stat_finish(acc, a.ws, a.stat);
}

template <bool STAT>
__global__ void __launch_bounds__(kThreads) agg_scalar_kernel(const AggArgs a)
{
    Acc3 acc = {0.0, 0.0, 0.0};
    for (unsigned long long i = (unsigned long long)blockIdx.x * kThreads + threadIdx.x; i < a.n;
         i += (unsigned long long)gridDim.x * kThreads)
        agg_elem<STAT>(a, i, acc);
    if (STAT) stat_finish(acc, a.ws, a.stat);
}

// ----------------------------------------------------------------------------------
// fused optimizer update + write-back + statistic
// ----------------------------------------------------------------------------------

struct UpdArgs {
    const float* g;                     // averaged gradient (two-kernel form) ...
    const float* gk[JABAS_MAX_VSW];     // ... or the kagg VSW gradients to aggregate on the fly
    float* gout;                        // fused form: nullable destination of the averaged gradient
    float divisor;                      // fused form: T
    int kagg;                           // 0: two-kernel form
    const float* grad_scale;            // nullable device scalar: g *= *grad_scale when it is < 1 (norm clipping)
    float* w[JABAS_MAX_VSW];
    float* m;
    float* v;
    const float* half;   // nullable
    double* stat;
    StatWs ws;
    const SegDev* segs;  // nullable: one group
    unsigned long long n, base;
    int nseg;
    int K;
    float half_divisor;
    const UpdHp* dyn;         // nullable: hyper-parameters live in device memory (CUDA-graph replay)
    int no_bulk;              // a gradient source is another GPU's memory: per-thread loads only
    // bulk-staged form only: pipeline depth, stream slots per stage (sized for the launch's
    // largest stream count) and the device counter of waits that ran out
    int stages, stage_slots;
    unsigned int* timeouts;
    unsigned long long wait_ns;   // wall-time limit of one wait for a stage's copies
    unsigned int extra_tx;        // test seam: bytes a stage's barrier expects beyond what is copied
    UpdHp hp;                 // ... otherwise they travel in the argument block
};

template <bool STAT>
__device__ __forceinline__ void half_stat4(const UpdArgs& a, float4 g, float4 hs, Acc3& acc)
{
    if (!STAT) return;
    const float4 e = div4(hs, a.half_divisor);
    const float4 o = make_float4(__fmaf_rn(2.0f, g.x, -e.x), __fmaf_rn(2.0f, g.y, -e.y),
                                 __fmaf_rn(2.0f, g.z, -e.z), __fmaf_rn(2.0f, g.w, -e.w));
    acc_vec(acc, e, o);
}

// Per-element form (tail, unaligned path, tiles that straddle a segment boundary).
template <int OPT, bool STAT>
__device__ __forceinline__ void upd_elem(const UpdArgs& a, const UpdHp& H, unsigned long long i, int seg,
                                         Acc3& acc)
{
    int gi = 0;
    if (a.segs) {
        while (__ldg(&a.segs[seg].end) <= a.base + i) ++seg;
        gi = (int)__ldg(&a.segs[seg].group);
    }
    float g, pe = 0.0f, po = 0.0f;
    if (a.kagg > 0) {                   // aggregate the VSW gradients, ascending k
        float s = a.gk[0][i];
        pe = s;
        for (int k = 1; k < a.kagg; ++k) {
            const float x = a.gk[k][i];
            s = __fadd_rn(s, x);
            if (k == 1) po = x;
            else if (k & 1) po = __fadd_rn(po, x);
            else pe = __fadd_rn(pe, x);
        }
        g = __fdiv_rn(s, a.divisor);
        if (a.gout) a.gout[i] = g;
    } else {
        g = a.g[i];
    }
    const float g_unclipped = g;
    if (a.grad_scale) {
        const float gs = __ldg(a.grad_scale);
        if (gs < 1.0f) g = __fmul_rn(g, gs);
    }
    float p = a.w[0][i];
    float m = (OPT == OPT_ADAM || ((H.flags & F_MOMENTUM) && !(H.flags & F_FIRST))) ? a.m[i] : 0.0f;
    float v = OPT == OPT_ADAM ? a.v[i] : 0.0f;
    upd_math<OPT>(H, H.grp[gi], (H.wd_mask >> gi) & 1u, g, p, m, v);
    for (int k = 0; k < a.K; ++k) a.w[k][i] = p;
    if (OPT == OPT_ADAM || (H.flags & F_MOMENTUM)) a.m[i] = m;
    if (OPT == OPT_ADAM) a.v[i] = v;
    if (STAT) {
        if (a.kagg > 0) {
            acc_one(acc, __fdiv_rn(pe, a.half_divisor), __fdiv_rn(po, a.half_divisor));
        } else {
            const float e = __fdiv_rn(a.half[i], a.half_divisor);
            acc_one(acc, e, __fmaf_rn(2.0f, g_unclipped, -e));
        }
    }
}

// Hyper-parameters of this launch into shared memory: from the argument block, or from the
// device-resident block when the launch is part of a replayed CUDA graph.
__device__ __forceinline__ void load_hp(const UpdArgs& a, UpdHp& H)
{
    if (a.dyn) {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(a.dyn);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&H);
        for (unsigned int i = threadIdx.x; i < sizeof(UpdHp) / 4; i += blockDim.x) dst[i] = __ldg(src + i);
    } else if (threadIdx.x == 0) {
        H = a.hp;
    }
    __syncthreads();
}

// KAGG = 0: g is read from a.g.  KAGG > 0 (single-GPU form): the KAGG VSW gradients are
// summed in registers (ascending k), divided by T and consumed at once, so the averaged
// gradient never makes a round trip through HBM; the statistic then comes from the
// even-/odd-VSW partial sums that are in registers anyway.
// Resident CTAs per SM asked of the compiler.  Measured on B200 (2^24..2^29 elements), two
// tiles per thread throughout K <= 4: with up to two gradient streams the kernel needs the
// third CTA per SM to cover its latency (K = 2: +23 % over 2 CTAs/SM at 118 registers);
// K = 3 and 4 are 3-7 % faster at 2 CTAs/SM with the registers that takes (K = 4 would
// spill at 80); from K = 5 one tile per thread at 3 CTAs/SM is 1 % ahead.
__host__ __device__ constexpr int upd_min_ctas(int KAGG) { return (KAGG == 3 || KAGG == 4) ? 1 : 3; }

// BULK: the inputs of a tile reach the registers through shared memory, staged by bulk
// copies (one 4 KB copy per stream and stage, `stages` tiles in flight per CTA) instead of
// per-thread 128-bit loads; U is 1.  Everything after the loads is the same code.
template <int OPT, bool STAT, int U, int KAGG, bool BULK>
__global__ void __launch_bounds__(kThreads, BULK ? 3 : upd_min_ctas(KAGG)) upd_vec_kernel(const UpdArgs a)
{
    static_assert(!BULK || U == 1, "the bulk-staged form handles one 4-vector per thread and tile");
    constexpr int KX = KAGG > 0 ? KAGG : 1;
    const float gscale = a.grad_scale ? __ldg(a.grad_scale) : 1.0f;
    const bool clip = gscale < 1.0f;
    const unsigned long long nvec = a.n >> 2;
    const unsigned long long tile = (unsigned long long)kThreads * U;
    __shared__ UpdHp H;
    extern __shared__ __align__(128) unsigned char stage_raw[];
    __shared__ unsigned long long stage_full[kMaxStages];
    bool stage_abort = false;     // decided per tile by a CTA-wide vote: the same in every thread
    if (BULK && threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) mbar_init(&stage_full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    load_hp(a, H);
    const bool use_m = OPT == OPT_ADAM || (H.flags & F_MOMENTUM);
    const bool load_m = OPT == OPT_ADAM || ((H.flags & F_MOMENTUM) && !(H.flags & F_FIRST));
    // slots of a stage: gradients (KX), p, then m / v / half as far as this launch reads them
    const int slot_m = KX + 1;
    const int slot_v = slot_m + (load_m ? 1 : 0);
    const int slot_h = slot_v + (OPT == OPT_ADAM ? 1 : 0);
    const unsigned long long my_first = (unsigned long long)blockIdx.x * tile;
    const unsigned long long stride = (unsigned long long)gridDim.x * tile;
    // thread 0 only: start the copies of the tile that begins at 4-vector t into stage s
    auto stage_issue = [&](unsigned long long t, int s) {
        const unsigned long long left = nvec - t;
        const unsigned bytes = left >= (unsigned long long)kStageTileVecs ? kStageTileBytes : (unsigned)left * 16u;
        const int nslot = slot_h + ((STAT && KAGG == 0) ? 1 : 0);
        unsigned char* sb = stage_raw + (size_t)s * a.stage_slots * kStageTileBytes;
        mbar_expect_tx(&stage_full[s], bytes * (unsigned)nslot + a.extra_tx);
        if (KAGG > 0) {
#pragma unroll
            for (int k = 0; k < KX; ++k) bulk_load(sb + k * kStageTileBytes, a.gk[k] + 4 * t, bytes, &stage_full[s]);
        } else {
            bulk_load(sb, a.g + 4 * t, bytes, &stage_full[s]);
        }
        bulk_load(sb + KX * kStageTileBytes, a.w[0] + 4 * t, bytes, &stage_full[s]);
        if (load_m) bulk_load(sb + slot_m * kStageTileBytes, a.m + 4 * t, bytes, &stage_full[s]);
        if (OPT == OPT_ADAM) bulk_load(sb + slot_v * kStageTileBytes, a.v + 4 * t, bytes, &stage_full[s]);
        if (STAT && KAGG == 0) bulk_load(sb + slot_h * kStageTileBytes, a.half + 4 * t, bytes, &stage_full[s]);
    };
    if (BULK && threadIdx.x == 0) {
        unsigned long long t = my_first;
        for (int s = 0; s < a.stages && t < nvec; ++s, t += stride) stage_issue(t, s);
    }
    Acc3 acc = {0.0, 0.0, 0.0};
    int cur_stage = 0;            // stage and mbarrier phase parity of the tile being consumed
    unsigned cur_parity = 0;
    unsigned long long t0 = my_first;
    for (; t0 < nvec; t0 += stride) {
        const bool full = t0 + tile <= nvec;
        float4 g[U], p[U], m[U], v[U], hs[U], xk[U][KX];
        if (BULK) {
            const int s = cur_stage;
            const bool landed = mbar_wait_bounded(&stage_full[s], cur_parity, a.wait_ns);
            const float4* sb = reinterpret_cast<const float4*>(stage_raw + (size_t)s * a.stage_slots * kStageTileBytes);
            m[0] = v[0] = hs[0] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (full || t0 + threadIdx.x < nvec) {
                if (KAGG > 0) {
#pragma unroll
                    for (int k = 0; k < KX; ++k) xk[0][k] = sb[k * kStageTileVecs + threadIdx.x];
                } else {
                    g[0] = sb[threadIdx.x];
                }
                p[0] = sb[KX * kStageTileVecs + threadIdx.x];
                if (load_m) m[0] = sb[slot_m * kStageTileVecs + threadIdx.x];
                if (OPT == OPT_ADAM) v[0] = sb[slot_v * kStageTileVecs + threadIdx.x];
                if (STAT && KAGG == 0) hs[0] = sb[slot_h * kStageTileVecs + threadIdx.x];
            }
            // the stage has been read by every thread; one vote per tile, so that all threads
            // leave the loop at the same tile when any thread's wait ran out
            if (__syncthreads_or(!landed)) { stage_abort = true; break; }
            if (threadIdx.x == 0) {
                const unsigned long long nt = t0 + (unsigned long long)a.stages * stride;
                if (nt < nvec) { fence_proxy_async_smem(); stage_issue(nt, s); }
            }
            if (++cur_stage == a.stages) { cur_stage = 0; cur_parity ^= 1u; }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long x = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                m[u] = v[u] = hs[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (full || x < nvec) {
                    if (KAGG > 0) {
#pragma unroll
                        for (int k = 0; k < KX; ++k) xk[u][k] = ld4(a.gk[k] + 4 * x);
                    } else {
                        g[u] = ld4(a.g + 4 * x);
                    }
                    p[u] = ld4(a.w[0] + 4 * x);
                    if (load_m) m[u] = ld4(a.m + 4 * x);
                    if (OPT == OPT_ADAM) v[u] = ld4(a.v + 4 * x);
                    if (STAT && KAGG == 0) hs[u] = ld4(a.half + 4 * x);
                }
            }
        }
        // segment of the tile's first element, uniform over the CTA: looked up here, before the
        // first use of the tile's data, so that the search runs while the loads are in flight
        int seg0 = 0, gi0 = 0;
        bool uniform = true;
        if (a.segs) {
            const unsigned long long e0 = a.base + 4 * t0;
            unsigned long long e1 = a.base + 4 * (t0 + tile);
            if (e1 > a.base + a.n) e1 = a.base + a.n;
            seg0 = seg_find(a.segs, a.nseg, e0);
            uniform = __ldg(&a.segs[seg0].end) >= e1;
            gi0 = (int)__ldg(&a.segs[seg0].group);
        }
        if (KAGG > 0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long x = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (!(full || x < nvec)) continue;
                float4 s = xk[u][0];
#pragma unroll
                for (int k = 1; k < KX; ++k) s = add4(s, xk[u][k]);
                g[u] = div4(s, a.divisor);
                if (a.gout) st4(a.gout + 4 * x, g[u]);
                if (STAT) {
                    float4 e = xk[u][0];
                    float4 o = xk[u][KX > 1 ? 1 : 0];
#pragma unroll
                    for (int k = 2; k < KX; ++k) {
                        if (k & 1) o = add4(o, xk[u][k]); else e = add4(e, xk[u][k]);
                    }
                    acc_vec(acc, div4(e, a.half_divisor), div4(o, a.half_divisor));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned long long x = t0 + (unsigned long long)u * kThreads + threadIdx.x;
            if (!(full || x < nvec)) continue;
            half_stat4<(STAT && KAGG == 0)>(a, g[u], hs[u], acc);
            if (clip)
                g[u] = make_float4(__fmul_rn(g[u].x, gscale), __fmul_rn(g[u].y, gscale),
                                   __fmul_rn(g[u].z, gscale), __fmul_rn(g[u].w, gscale));
            if (uniform) {
                upd_math4<OPT>(H, H.grp[gi0], (H.wd_mask >> gi0) & 1u, g[u], p[u], m[u], v[u]);
            } else {
                int s = seg0;
                auto one = [&](int c, float gx, float& px, float& mx, float& vx) {
                    while (__ldg(&a.segs[s].end) <= a.base + 4 * x + c) ++s;
                    const int gi = (int)__ldg(&a.segs[s].group);
                    upd_math<OPT>(H, H.grp[gi], (H.wd_mask >> gi) & 1u, gx, px, mx, vx);
                };
                one(0, g[u].x, p[u].x, m[u].x, v[u].x);
                one(1, g[u].y, p[u].y, m[u].y, v[u].y);
                one(2, g[u].z, p[u].z, m[u].z, v[u].z);
                one(3, g[u].w, p[u].w, m[u].w, v[u].w);
            }
            for (int k = 0; k < a.K; ++k) st4(a.w[k] + 4 * x, p[u]);
            if (use_m) st4(a.m + 4 * x, m[u]);
            if (OPT == OPT_ADAM) st4(a.v + 4 * x, v[u]);
        }
    }
    if (BULK && stage_abort) {
        // a wait ran out: report it, and give the copies still in flight one more bounded
        // wait each so that none lands in shared memory after the CTA has gone
        // (t0, cur_stage, cur_parity still describe the tile whose wait failed)
        unsigned long long t = t0;
        for (int j = 0; j < a.stages && t < nvec; ++j, t += stride) {
            (void)mbar_wait_bounded(&stage_full[cur_stage], cur_parity, a.wait_ns);
            if (++cur_stage == a.stages) { cur_stage = 0; cur_parity ^= 1u; }
        }
        if (threadIdx.x == 0 && a.timeouts) atomicAdd(a.timeouts, 1u);
    }
    const unsigned int rem = (unsigned int)(a.n & 3ull);
    if (blockIdx.x == 0 && threadIdx.x < rem) {
        const unsigned long long i = (nvec << 2) + threadIdx.x;
        upd_elem<OPT, STAT>(a, H, i, a.segs ? seg_find(a.segs, a.nseg, a.base + i) : 0, acc);
    }
    if (STAT) stat_finish(acc, a.ws, a.stat);
}

template <int OPT, bool STAT>
__global__ void __launch_bounds__(kThreads) upd_scalar_kernel(const UpdArgs a)
{
    __shared__ UpdHp H;
    load_hp(a, H);
    Acc3 acc = {0.0, 0.0, 0.0};
    for (unsigned long long i = (unsigned long long)blockIdx.x * kThreads + threadIdx.x; i < a.n;
         i += (unsigned long long)gridDim.x * kThreads)
        upd_elem<OPT, STAT>(a, H, i, a.segs ? seg_find(a.segs, a.nseg, a.base + i) : 0, acc);
    if (STAT) stat_finish(acc, a.ws, a.stat);
}

// ----------------------------------------------------------------------------------
// small kernels: in-place division, dot/norms, finalize, replicate
// ----------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads) div_kernel(float* x, unsigned long long n, float d, int vec)
{
    const unsigned long long tid = (unsigned long long)blockIdx.x * kThreads + threadIdx.x;
    const unsigned long long stride = (unsigned long long)gridDim.x * kThreads;
    if (vec) {
        const unsigned long long nvec = n >> 2;
        for (unsigned long long i = tid; i < nvec; i += stride) st4(x + 4 * i, div4(ld4(x + 4 * i), d));
        if (tid < (n & 3ull)) x[(nvec << 2) + tid] = __fdiv_rn(x[(nvec << 2) + tid], d);
    } else {
        for (unsigned long long i = tid; i < n; i += stride) x[i] = __fdiv_rn(x[i], d);
    }
}

template <bool ONE>   // ONE: b is a, read once (sum of squares)
__global__ void __launch_bounds__(kThreads) dot_norms_kernel(const float* a, const float* b,
                                                             unsigned long long n, int vec,
                                                             StatWs ws, double* stat)
{
    constexpr int U = 4;
    Acc3 acc = {0.0, 0.0, 0.0};
    if (vec) {
        const unsigned long long nvec = n >> 2;
        const unsigned long long tile = (unsigned long long)kThreads * U;
        for (unsigned long long t0 = (unsigned long long)blockIdx.x * tile; t0 < nvec;
             t0 += (unsigned long long)gridDim.x * tile) {
            float4 x[U], y[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long i = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                x[u] = y[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < nvec) { x[u] = ld4(a + 4 * i); y[u] = ONE ? x[u] : ld4(b + 4 * i); }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) acc_vec(acc, x[u], y[u]);
        }
        if (blockIdx.x == 0 && threadIdx.x < (n & 3ull)) {
            const unsigned long long i = (nvec << 2) + threadIdx.x;
            acc_one(acc, a[i], b[i]);
        }
    } else {
        for (unsigned long long i = (unsigned long long)blockIdx.x * kThreads + threadIdx.x; i < n;
             i += (unsigned long long)gridDim.x * kThreads)
            acc_one(acc, a[i], b[i]);
    }
    stat_finish(acc, ws, stat);
}

__global__ void cosine_finalize_kernel(const double* stat, double eps, float* out)
{
    double den = stat[1] * stat[2];
    if (den < eps * eps) den = eps * eps;
    out[0] = (float)(stat[0] / sqrt(den));
}

// torch.nn.utils.clip_grad_norm_ of PyTorch v1.8.1 on the fp64 sum of squares:
// total_norm = sqrt(sumsq) as fp32, clip_coef = max_norm / (total_norm + 1e-6) in fp32.
__global__ void clip_coef_kernel(const double* sumsq, float max_norm, float* out)
{
    const float total = (float)sqrt(sumsq[0]);
    out[0] = __fdiv_rn(max_norm, __fadd_rn(total, 1e-6f));
    out[1] = total;
}

struct RepArgs {
    const float* src;
    float* dst[JABAS_MAX_VSW];
    int ndst;
    int vec;
    unsigned long long n;
};

__global__ void __launch_bounds__(kThreads) replicate_kernel(const RepArgs a)
{
    constexpr int U = 4;
    if (a.vec) {
        const unsigned long long nvec = a.n >> 2;
        const unsigned long long tile = (unsigned long long)kThreads * U;
        for (unsigned long long t0 = (unsigned long long)blockIdx.x * tile; t0 < nvec;
             t0 += (unsigned long long)gridDim.x * tile) {
            float4 x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long i = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (i < nvec) x[u] = ld4(a.src + 4 * i);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long i = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (i < nvec)
                    for (int k = 0; k < a.ndst; ++k) st4(a.dst[k] + 4 * i, x[u]);
            }
        }
        if (blockIdx.x == 0 && threadIdx.x < (a.n & 3ull)) {
            const unsigned long long i = (nvec << 2) + threadIdx.x;
            for (int k = 0; k < a.ndst; ++k) a.dst[k][i] = a.src[i];
        }
    } else {
        for (unsigned long long i = (unsigned long long)blockIdx.x * kThreads + threadIdx.x; i < a.n;
             i += (unsigned long long)gridDim.x * kThreads)
            for (int k = 0; k < a.ndst; ++k) a.dst[k][i] = a.src[i];
    }
}

// ----------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------

}  // namespace

int jb_ctx_bind(jabas_ctx_t* ctx)
{
    if (!ctx) return fail(JABAS_EINVAL, "ctx is null");
    int cur = -1;
    JB_CUDA(cudaGetDevice(&cur));
    if (cur != ctx->device) JB_CUDA(cudaSetDevice(ctx->device));
    return JABAS_OK;
}

namespace {

inline int ctx_bind(jabas_ctx_t* ctx) { return jb_ctx_bind(ctx); }

// Resident CTAs per SM of a kernel, cached per context.
template <typename KernelT>
int grid_for(jabas_ctx_t* ctx, KernelT kernel, unsigned long long work_items, unsigned long long per_cta,
             int* grid, size_t dyn_smem = 0)
{
    // kernels that take dynamic shared memory (the bulk-staged forms) never ask for more than
    // kStageBudgetBytes: the occupancy is computed once, for that budget, and cached per kernel
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lk(ctx->mu);
        auto it = ctx->occ.find(reinterpret_cast<const void*>(kernel));
        if (it != ctx->occ.end()) per_sm = it->second;
    }
    if (per_sm == 0) {
        if (dyn_smem > 0)
            JB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBudgetBytes));
        JB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads,
                                                              dyn_smem > 0 ? (size_t)kStageBudgetBytes : 0));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
        std::lock_guard<std::mutex> lk(ctx->mu);
        ctx->occ[reinterpret_cast<const void*>(kernel)] = per_sm;
    }
    unsigned long long need = (work_items + per_cta - 1) / per_cta;
    if (need < 1) need = 1;
    const unsigned long long cap = (unsigned long long)ctx->sm_count * per_sm;
    *grid = (int)(need < cap ? need : cap);
    return JABAS_OK;
}

int ws_for(jabas_ctx_t* ctx, void* stream, StatWs* out)
{
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->ws.find(stream);
    if (it != ctx->ws.end()) { *out = it->second; return JABAS_OK; }
    StatWs w{};
    char* raw = nullptr;
    const size_t bytes = 256 + sizeof(double) * 3 * (size_t)ctx->max_grid;
    JB_CUDA(cudaMalloc(&raw, bytes));
    cudaError_t e = cudaMemset(raw, 0, bytes);
    if (e != cudaSuccess) { cudaFree(raw); return fail(JABAS_ECUDA, cudaGetErrorString(e)); }
    w.counter = reinterpret_cast<unsigned int*>(raw);
    w.partials = reinterpret_cast<double*>(raw + 256);
    ctx->ws[stream] = w;
    *out = w;
    return JABAS_OK;
}

template <int K>
struct AggLaunch {
    static int run(jabas_ctx_t* ctx, const AggArgs& a, cudaStream_t st)
    {
        constexpr int U = agg_unroll(K);
        int grid = 0, rc;
        if (a.stat) {
            if ((rc = grid_for(ctx, agg_vec_kernel<K, true>, a.n >> 2, (unsigned long long)kThreads * U, &grid))) return rc;
            agg_vec_kernel<K, true><<<grid, kThreads, 0, st>>>(a);
        } else {
            if ((rc = grid_for(ctx, agg_vec_kernel<K, false>, a.n >> 2, (unsigned long long)kThreads * U, &grid))) return rc;
            agg_vec_kernel<K, false><<<grid, kThreads, 0, st>>>(a);
        }
        return JABAS_OK;
    }
};

template <int K>
int agg_dispatch(jabas_ctx_t* ctx, const AggArgs& a, cudaStream_t st)
{
    if (a.K == K) return AggLaunch<K>::run(ctx, a, st);
    if constexpr (K < JABAS_MAX_VSW) return agg_dispatch<K + 1>(ctx, a, st);
    return fail(JABAS_EINVAL, "K out of range");
}

constexpr int kMaxFusedVsw = 8;     // the fused aggregate+update form is instantiated for K <= 8

// Stages of the bulk-staged form: as many tiles in flight as fit the shared-memory budget.
inline int stage_count(int slots)
{
    int s = kStageBudgetBytes / (slots * (int)kStageTileBytes);
    return s < 1 ? 1 : (s > kMaxStages ? kMaxStages : s);
}

template <int OPT, int KAGG>
int upd_launch_vec(jabas_ctx_t* ctx, UpdArgs& a, cudaStream_t st)
{
    if (a.kagg != KAGG) {
        if constexpr (KAGG < kMaxFusedVsw) return upd_launch_vec<OPT, KAGG + 1>(ctx, a, st);
        return fail(JABAS_EINVAL, "fused aggregate+update supports at most 8 VSWs");
    }
    int grid = 0, rc;
    if (ctx->staging == JABAS_STAGING_BULK && !a.no_bulk) {
        // slots for the launch's largest stream count: gradients, p, m [, v] [, half]
        a.stage_slots = (KAGG > 0 ? KAGG : 1) + 2 + (OPT == OPT_ADAM ? 1 : 0) + ((a.stat && KAGG == 0) ? 1 : 0);
        a.stages = stage_count(a.stage_slots);
        a.timeouts = ctx->d_timeouts;
        a.wait_ns = (unsigned long long)(ctx->staging_wait_ms * 1e6);
        a.extra_tx = ctx->stall_tx;
        const size_t smem = (size_t)a.stages * a.stage_slots * kStageTileBytes;
        if (a.stat) {
            if ((rc = grid_for(ctx, upd_vec_kernel<OPT, true, 1, KAGG, true>, a.n >> 2, kThreads, &grid, smem))) return rc;
            upd_vec_kernel<OPT, true, 1, KAGG, true><<<grid, kThreads, smem, st>>>(a);
        } else {
            if ((rc = grid_for(ctx, upd_vec_kernel<OPT, false, 1, KAGG, true>, a.n >> 2, kThreads, &grid, smem))) return rc;
            upd_vec_kernel<OPT, false, 1, KAGG, true><<<grid, kThreads, smem, st>>>(a);
        }
        return JABAS_OK;
    }
    constexpr int U = KAGG > 4 ? 1 : 2;
    if (a.stat) {
        if ((rc = grid_for(ctx, upd_vec_kernel<OPT, true, U, KAGG, false>, a.n >> 2, (unsigned long long)kThreads * U, &grid))) return rc;
        upd_vec_kernel<OPT, true, U, KAGG, false><<<grid, kThreads, 0, st>>>(a);
    } else {
        if ((rc = grid_for(ctx, upd_vec_kernel<OPT, false, U, KAGG, false>, a.n >> 2, (unsigned long long)kThreads * U, &grid))) return rc;
        upd_vec_kernel<OPT, false, U, KAGG, false><<<grid, kThreads, 0, st>>>(a);
    }
    return JABAS_OK;
}

template <int OPT>
int upd_launch(jabas_ctx_t* ctx, UpdArgs& a, bool vec, cudaStream_t st)
{
    int grid = 0, rc;
    if (vec) {
        if ((rc = upd_launch_vec<OPT, 0>(ctx, a, st))) return rc;
    } else {
        if (a.stat) {
            if ((rc = grid_for(ctx, upd_scalar_kernel<OPT, true>, a.n, kThreads, &grid))) return rc;
            upd_scalar_kernel<OPT, true><<<grid, kThreads, 0, st>>>(a);
        } else {
            if ((rc = grid_for(ctx, upd_scalar_kernel<OPT, false>, a.n, kThreads, &grid))) return rc;
            upd_scalar_kernel<OPT, false><<<grid, kThreads, 0, st>>>(a);
        }
    }
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

// Where the gradient of an update comes from: one averaged buffer, or K VSW buffers that the
// kernel aggregates itself (single-GPU form).
struct GradSrc {
    const float* g;
    const float* const* grads;
    int kg;
    float divisor;
    float* gout;
};

// Validation and argument marshalling shared by the two optimizers.
int upd_prepare(jabas_ctx_t* ctx, UpdArgs& a, bool* vec, const GradSrc& src, float* const* w, int K,
                float* m, float* v, uint64_t n, uint64_t base, const jabas_layout_t* layout,
                const jabas_group_t* groups, int ngroups, const float* half, float half_divisor,
                double* stat3, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!w) return fail(JABAS_EINVAL, "w is null");
    if (K < 1 || K > JABAS_MAX_VSW) return fail(JABAS_EINVAL, "K must be in [1, JABAS_MAX_VSW]");
    const bool fused = src.grads != nullptr;
    if (fused) {
        if (src.kg < 1 || src.kg > kMaxFusedVsw)
            return fail(JABAS_EINVAL, "fused aggregate+update supports 1..8 VSW gradients");
        if (!(src.divisor != 0.0f)) return fail(JABAS_EINVAL, "divisor must be non-zero");
        if (half) return fail(JABAS_EINVAL, "the fused form takes its statistic from the VSW gradients, not from half");
        if (stat3 && (src.kg < 2 || !(half_divisor != 0.0f)))
            return fail(JABAS_EINVAL, "the VSW-parity statistic needs K >= 2 and a non-zero half_divisor");
    }
    if (!groups || ngroups < 1 || ngroups > JABAS_MAX_GROUPS)
        return fail(JABAS_EINVAL, "ngroups must be in [1, JABAS_MAX_GROUPS]");
    if (!fused && (half == nullptr) != (stat3 == nullptr))
        return fail(JABAS_EINVAL, "half and stat3 must both be set or both be null");
    if (half && !(half_divisor != 0.0f)) return fail(JABAS_EINVAL, "half_divisor must be non-zero");
    std::memset(&a, 0, sizeof(a));
    a.g = src.g; a.m = m; a.v = v; a.half = half; a.stat = stat3;
    a.n = n; a.base = base; a.K = K; a.half_divisor = half_divisor;
    *vec = (!m || aligned16(m)) && (!v || aligned16(v)) && (!half || aligned16(half));
    if (fused) {
        a.kagg = src.kg; a.divisor = src.divisor; a.gout = src.gout;
        *vec = *vec && (!src.gout || aligned16(src.gout));
        for (int k = 0; k < src.kg; ++k) {
            if (!src.grads[k]) return fail(JABAS_EINVAL, "grads[k] is null");
            a.gk[k] = src.grads[k];
            *vec = *vec && aligned16(src.grads[k]);
        }
    } else {
        *vec = *vec && (!src.g || aligned16(src.g));
    }
    for (int k = 0; k < K; ++k) {
        if (!w[k]) return fail(JABAS_EINVAL, "w[k] is null");
        a.w[k] = w[k];
        *vec = *vec && aligned16(w[k]);
    }
    if (layout) {
        if (layout->device != ctx->device) return fail(JABAS_EINVAL, "layout belongs to another device");
        if (base + n > layout->total) return fail(JABAS_EINVAL, "base + n exceeds the layout");
        if (layout->max_group >= ngroups)
            return fail(JABAS_EINVAL, "the layout names a param group that the call does not provide");
        a.segs = layout->dsegs; a.nseg = layout->nseg;
    }
    if (stat3 && (rc = ws_for(ctx, stream, &a.ws))) return rc;
    return JABAS_OK;
}

}  // namespace

// Host -> kernel form of the hyper-parameters: fp64 scalars rounded to fp32 once.
int jb_fill_sgd_hp(UpdHp& h, const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* hp)
{
    std::memset(&h, 0, sizeof(h));
    h.c0 = (float)hp->momentum;
    h.c1 = (float)(1.0 - hp->dampening);
    h.flags = (hp->nesterov ? F_NESTEROV : 0u) | (hp->first_step ? F_FIRST : 0u) |
              (hp->momentum != 0.0 ? F_MOMENTUM : 0u);
    for (int i = 0; i < ngroups; ++i) {
        h.grp[i].wd = (float)groups[i].weight_decay;
        h.grp[i].s0 = (float)(-groups[i].lr);
        if (groups[i].weight_decay != 0.0) h.wd_mask |= 1u << i;
    }
    return JABAS_OK;
}

int jb_fill_adam_hp(UpdHp& h, const jabas_group_t* groups, int ngroups, const jabas_adam_hp_t* hp)
{
    std::memset(&h, 0, sizeof(h));
    h.c0 = (float)hp->beta1; h.c1 = (float)hp->beta2;
    h.c2 = (float)(1.0 - hp->beta1); h.c3 = (float)(1.0 - hp->beta2);
    h.c4 = (float)hp->eps;
    h.flags = hp->decoupled ? F_DECOUPLED : 0u;
    for (int i = 0; i < ngroups; ++i) {
        if (groups[i].step < 1) return fail(JABAS_EINVAL, "Adam step must be >= 1");
        const double bc1 = 1.0 - std::pow(hp->beta1, (double)groups[i].step);
        const double bc2 = 1.0 - std::pow(hp->beta2, (double)groups[i].step);
        h.grp[i].wd = (float)groups[i].weight_decay;
        h.grp[i].s0 = (float)(1.0 - groups[i].lr * groups[i].weight_decay);
        h.grp[i].s1 = (float)(-(groups[i].lr / bc1));
        h.grp[i].s2 = (float)std::sqrt(bc2);
        if (groups[i].weight_decay != 0.0) h.wd_mask |= 1u << i;
    }
    return JABAS_OK;
}

extern "C" {

int jabas_version(void) { return JABAS_B200_VERSION; }

const char* jabas_last_error(void) { return g_err.c_str(); }

int jabas_ctx_create(int device, jabas_ctx_t** out)
{
    if (!out) return fail(JABAS_EINVAL, "ctx out pointer is null");
    *out = nullptr;
    int count = 0;
    JB_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(JABAS_EINVAL, "no such CUDA device");
    jabas_ctx_t* c = new (std::nothrow) jabas_ctx_t();
    if (!c) return fail(JABAS_ENOMEM, "out of host memory");
    c->device = device;
    cudaError_t e = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) { delete c; return fail(JABAS_ECUDA, cudaGetErrorString(e)); }
    c->max_grid = c->sm_count * kMaxCtasPerSm;
    *out = c;
    return JABAS_OK;
}

int jabas_ctx_destroy(jabas_ctx_t* ctx)
{
    if (!ctx) return JABAS_OK;
    int rc = ctx_bind(ctx);
    if (rc == JABAS_OK) {
        for (auto& kv : ctx->ws) cudaFree(kv.second.counter);
        if (ctx->d_timeouts) cudaFree(ctx->d_timeouts);
    }
    delete ctx;
    return rc;
}

int jabas_ctx_set_staging(jabas_ctx_t* ctx, int mode)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (mode != JABAS_STAGING_REGISTER && mode != JABAS_STAGING_BULK)
        return fail(JABAS_EINVAL, "staging mode must be JABAS_STAGING_REGISTER or JABAS_STAGING_BULK");
    if (mode == JABAS_STAGING_BULK && !ctx->d_timeouts) {
        unsigned int* d = nullptr;
        if (cudaMalloc(&d, sizeof(unsigned int)) != cudaSuccess) return fail(JABAS_ENOMEM, "out of device memory");
        cudaError_t e = cudaMemset(d, 0, sizeof(unsigned int));
        if (e != cudaSuccess) { cudaFree(d); return fail(JABAS_ECUDA, cudaGetErrorString(e)); }
        ctx->d_timeouts = d;
    }
    ctx->staging = mode;
    return JABAS_OK;
}

int jabas_ctx_set_wait_limits(jabas_ctx_t* ctx, double staging_ms, double peer_ms)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!(staging_ms > 0.0) || !(peer_ms > 0.0) || staging_ms > 60e3 || peer_ms > 60e3)
        return fail(JABAS_EINVAL, "wait limits must be in (0, 60000] milliseconds");
    ctx->staging_wait_ms = staging_ms;
    ctx->peer_wait_ms = peer_ms;
    return JABAS_OK;
}

int jabas_ctx_inject_staging_stall(jabas_ctx_t* ctx, int on)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    ctx->stall_tx = on ? 16u : 0u;
    return JABAS_OK;
}

int jabas_ctx_staging_timeouts(jabas_ctx_t* ctx, uint32_t* count)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!count) return fail(JABAS_EINVAL, "count is null");
    *count = 0;
    if (!ctx->d_timeouts) return JABAS_OK;
    unsigned int h = 0;
    JB_CUDA(cudaMemcpy(&h, ctx->d_timeouts, sizeof(h), cudaMemcpyDeviceToHost));
    *count = h;
    return JABAS_OK;
}

int jabas_layout_create(jabas_ctx_t* ctx, const jabas_seg_t* segs, int nseg, uint64_t total,
                        jabas_layout_t** out)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!out) return fail(JABAS_EINVAL, "layout out pointer is null");
    *out = nullptr;
    if (!segs || nseg < 1) return fail(JABAS_EINVAL, "empty segment table");
    std::vector<SegDev> h((size_t)nseg);
    uint64_t pos = 0;
    int max_group = 0;
    for (int i = 0; i < nseg; ++i) {
        if (segs[i].begin != pos || segs[i].end <= segs[i].begin)
            return fail(JABAS_EINVAL, "segments must be sorted, non-empty and contiguous from 0");
        if (segs[i].group >= JABAS_MAX_GROUPS) return fail(JABAS_EINVAL, "segment group out of range");
        h[i].begin = segs[i].begin; h[i].end = segs[i].end; h[i].group = segs[i].group; h[i].pad = 0;
        pos = segs[i].end;
        if ((int)segs[i].group > max_group) max_group = (int)segs[i].group;
    }
    if (pos != total) return fail(JABAS_EINVAL, "segments do not cover [0, total)");
    jabas_layout_t* l = new (std::nothrow) jabas_layout_t();
    if (!l) return fail(JABAS_ENOMEM, "out of host memory");
    l->device = ctx->device; l->nseg = nseg; l->total = total; l->max_group = max_group;
    cudaError_t e = cudaMalloc(&l->dsegs, sizeof(SegDev) * (size_t)nseg);
    if (e == cudaSuccess) e = cudaMemcpy(l->dsegs, h.data(), sizeof(SegDev) * (size_t)nseg, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        if (l->dsegs) cudaFree(l->dsegs);
        delete l;
        return fail(JABAS_ECUDA, cudaGetErrorString(e));
    }
    *out = l;
    return JABAS_OK;
}

int jabas_layout_destroy(jabas_layout_t* layout)
{
    if (!layout) return JABAS_OK;
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != layout->device) cudaSetDevice(layout->device);
    cudaFree(layout->dsegs);
    delete layout;
    return JABAS_OK;
}

int jabas_vsw_aggregate_f32(jabas_ctx_t* ctx, const float* const* grads, int K, float* out,
                            float* half_out, uint64_t n, float divisor, float half_divisor,
                            double* stat3, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!grads || !out) return fail(JABAS_EINVAL, "grads or out is null");
    if (K < 1 || K > JABAS_MAX_VSW) return fail(JABAS_EINVAL, "K must be in [1, JABAS_MAX_VSW]");
    if (!(divisor != 0.0f)) return fail(JABAS_EINVAL, "divisor must be non-zero");
    if (stat3 && K < 2) return fail(JABAS_EINVAL, "the VSW-parity statistic needs K >= 2");
    if (stat3 && !(half_divisor != 0.0f)) return fail(JABAS_EINVAL, "half_divisor must be non-zero");
    if (n == 0) return JABAS_OK;
    AggArgs a;
    std::memset(&a, 0, sizeof(a));
    bool vec = aligned16(out) && (!half_out || aligned16(half_out));
    for (int k = 0; k < K; ++k) {
        if (!grads[k]) return fail(JABAS_EINVAL, "grads[k] is null");
        a.g[k] = grads[k];
        vec = vec && aligned16(grads[k]);
    }
    a.out = out; a.half = half_out; a.stat = stat3; a.n = n; a.divisor = divisor;
    a.half_divisor = half_divisor; a.K = K;
    if (stat3 && (rc = ws_for(ctx, stream, &a.ws))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec) {
        if ((rc = agg_dispatch<1>(ctx, a, st))) return rc;
    } else {
        int grid = 0;
        if (stat3) {
            if ((rc = grid_for(ctx, agg_scalar_kernel<true>, n, kThreads, &grid))) return rc;
            agg_scalar_kernel<true><<<grid, kThreads, 0, st>>>(a);
        } else {
            if ((rc = grid_for(ctx, agg_scalar_kernel<false>, n, kThreads, &grid))) return rc;
            agg_scalar_kernel<false><<<grid, kThreads, 0, st>>>(a);
        }
    }
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_div_f32(jabas_ctx_t* ctx, float* x, uint64_t n, float divisor, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!x) return fail(JABAS_EINVAL, "x is null");
    if (!(divisor != 0.0f)) return fail(JABAS_EINVAL, "divisor must be non-zero");
    if (n == 0) return JABAS_OK;
    const int vec = aligned16(x) ? 1 : 0;
    int grid = 0;
    if ((rc = grid_for(ctx, div_kernel, vec ? (n + 3) / 4 : n, kThreads, &grid))) return rc;
    div_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, n, divisor, vec);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

static int sgd_impl(jabas_ctx_t* ctx, const GradSrc& src, float* const* w, int K, float* m,
                    uint64_t n, uint64_t base, const jabas_layout_t* layout,
                    const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* hp,
                    const float* half, float half_divisor, double* stat3, void* stream)
{
    if (!hp) return fail(JABAS_EINVAL, "hp is null");
    UpdArgs a;
    bool vec = false;
    int rc = upd_prepare(ctx, a, &vec, src, w, K, m, nullptr, n, base, layout, groups, ngroups, half,
                         half_divisor, stat3, stream);
    if (rc) return rc;
    if (hp->momentum != 0.0 && !m) return fail(JABAS_EINVAL, "momentum != 0 needs a momentum buffer");
    if (hp->nesterov && (hp->momentum <= 0.0 || hp->dampening != 0.0))
        return fail(JABAS_EINVAL, "nesterov needs momentum > 0 and dampening == 0");
    if (n == 0) return JABAS_OK;
    a.grad_scale = hp->grad_scale;
    a.no_bulk = hp->remote_sources ? 1 : 0;
    if ((rc = jb_fill_sgd_hp(a.hp, groups, ngroups, hp))) return rc;
    if (hp->dynamic) {
        if (hp->dynamic->kind != OPT_SGD) return fail(JABAS_EINVAL, "the dynamic block holds Adam hyper-parameters");
        a.dyn = hp->dynamic->dev;
    }
    return upd_launch<OPT_SGD>(ctx, a, vec, static_cast<cudaStream_t>(stream));
}

int jabas_sgd_momentum_f32(jabas_ctx_t* ctx, const float* g, float* const* w, int K, float* m,
                           uint64_t n, uint64_t base, const jabas_layout_t* layout,
                           const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* hp,
                           const float* half, float half_divisor, double* stat3, void* stream)
{
    const GradSrc src = {g, nullptr, 0, 1.0f, nullptr};
    if (!g) return fail(JABAS_EINVAL, "g is null");
    return sgd_impl(ctx, src, w, K, m, n, base, layout, groups, ngroups, hp, half, half_divisor, stat3, stream);
}

int jabas_vsw_sgd_momentum_f32(jabas_ctx_t* ctx, const float* const* grads, int Kg, float divisor,
                               float* grad_out, float* const* w, int K, float* m, uint64_t n,
                               uint64_t base, const jabas_layout_t* layout, const jabas_group_t* groups,
                               int ngroups, const jabas_sgd_hp_t* hp, float half_divisor, double* stat3,
                               void* stream)
{
    if (!grads) return fail(JABAS_EINVAL, "grads is null");
    const GradSrc src = {nullptr, grads, Kg, divisor, grad_out};
    return sgd_impl(ctx, src, w, K, m, n, base, layout, groups, ngroups, hp, nullptr, half_divisor, stat3, stream);
}

static int adam_impl(jabas_ctx_t* ctx, const GradSrc& src, float* const* w, int K, float* m, float* v,
                     uint64_t n, uint64_t base, const jabas_layout_t* layout,
                     const jabas_group_t* groups, int ngroups, const jabas_adam_hp_t* hp,
                     const float* half, float half_divisor, double* stat3, void* stream)
{
    if (!hp) return fail(JABAS_EINVAL, "hp is null");
    UpdArgs a;
    bool vec = false;
    int rc = upd_prepare(ctx, a, &vec, src, w, K, m, v, n, base, layout, groups, ngroups, half,
                         half_divisor, stat3, stream);
    if (rc) return rc;
    if (!m || !v) return fail(JABAS_EINVAL, "exp_avg and exp_avg_sq buffers are required");
    if (n == 0) return JABAS_OK;
    a.grad_scale = hp->grad_scale;
    a.no_bulk = hp->remote_sources ? 1 : 0;
    if ((rc = jb_fill_adam_hp(a.hp, groups, ngroups, hp))) return rc;
    if (hp->dynamic) {
        if (hp->dynamic->kind != OPT_ADAM) return fail(JABAS_EINVAL, "the dynamic block holds SGD hyper-parameters");
        a.dyn = hp->dynamic->dev;
    }
    return upd_launch<OPT_ADAM>(ctx, a, vec, static_cast<cudaStream_t>(stream));
}

int jabas_adam_f32(jabas_ctx_t* ctx, const float* g, float* const* w, int K, float* m, float* v,
                   uint64_t n, uint64_t base, const jabas_layout_t* layout,
                   const jabas_group_t* groups, int ngroups, const jabas_adam_hp_t* hp,
                   const float* half, float half_divisor, double* stat3, void* stream)
{
    const GradSrc src = {g, nullptr, 0, 1.0f, nullptr};
    if (!g) return fail(JABAS_EINVAL, "g is null");
    return adam_impl(ctx, src, w, K, m, v, n, base, layout, groups, ngroups, hp, half, half_divisor, stat3, stream);
}

int jabas_vsw_adam_f32(jabas_ctx_t* ctx, const float* const* grads, int Kg, float divisor, float* grad_out,
                       float* const* w, int K, float* m, float* v, uint64_t n, uint64_t base,
                       const jabas_layout_t* layout, const jabas_group_t* groups, int ngroups,
                       const jabas_adam_hp_t* hp, float half_divisor, double* stat3, void* stream)
{
    if (!grads) return fail(JABAS_EINVAL, "grads is null");
    const GradSrc src = {nullptr, grads, Kg, divisor, grad_out};
    return adam_impl(ctx, src, w, K, m, v, n, base, layout, groups, ngroups, hp, nullptr, half_divisor, stat3, stream);
}

int jabas_dynhp_create(jabas_ctx_t* ctx, jabas_dynhp_t** out)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!out) return fail(JABAS_EINVAL, "dynhp out pointer is null");
    *out = nullptr;
    jabas_dynhp_t* h = new (std::nothrow) jabas_dynhp_t();
    if (!h) return fail(JABAS_ENOMEM, "out of host memory");
    h->device = ctx->device;
    cudaError_t e = cudaMalloc(&h->dev, sizeof(UpdHp));
    if (e == cudaSuccess) e = cudaMemset(h->dev, 0, sizeof(UpdHp));
    if (e == cudaSuccess) e = cudaMallocHost(&h->pinned, sizeof(UpdHp) * jabas_dynhp::kSlots);
    for (int i = 0; e == cudaSuccess && i < jabas_dynhp::kSlots; ++i)
        e = cudaEventCreateWithFlags(&h->done[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
        jabas_dynhp_destroy(h);
        return fail(JABAS_ECUDA, cudaGetErrorString(e));
    }
    *out = h;
    return JABAS_OK;
}

int jabas_dynhp_destroy(jabas_dynhp_t* h)
{
    if (!h) return JABAS_OK;
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != h->device) cudaSetDevice(h->device);
    for (int i = 0; i < jabas_dynhp::kSlots; ++i)
        if (h->done[i]) cudaEventDestroy(h->done[i]);
    if (h->pinned) cudaFreeHost(h->pinned);
    if (h->dev) cudaFree(h->dev);
    delete h;
    return JABAS_OK;
}

static int dynhp_push(jabas_dynhp_t* h, const UpdHp& v, int kind, void* stream)
{
    std::lock_guard<std::mutex> lk(h->mu);
    int cur = -1;
    JB_CUDA(cudaGetDevice(&cur));
    if (cur != h->device) JB_CUDA(cudaSetDevice(h->device));
    const int slot = h->next;
    h->next = (slot + 1) % jabas_dynhp::kSlots;
    JB_CUDA(cudaEventSynchronize(h->done[slot]));      // the copy that last used this slot is over
    h->pinned[slot] = v;
    h->kind = kind;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    JB_CUDA(cudaMemcpyAsync(h->dev, h->pinned + slot, sizeof(UpdHp), cudaMemcpyHostToDevice, st));
    JB_CUDA(cudaEventRecord(h->done[slot], st));
    return JABAS_OK;
}

int jabas_dynhp_push_sgd(jabas_dynhp_t* h, const jabas_group_t* groups, int ngroups,
                         const jabas_sgd_hp_t* hp, void* stream)
{
    if (!h || !groups || !hp) return fail(JABAS_EINVAL, "null argument");
    if (ngroups < 1 || ngroups > JABAS_MAX_GROUPS) return fail(JABAS_EINVAL, "ngroups must be in [1, JABAS_MAX_GROUPS]");
    UpdHp v;
    int rc = jb_fill_sgd_hp(v, groups, ngroups, hp);
    return rc ? rc : dynhp_push(h, v, OPT_SGD, stream);
}

int jabas_dynhp_push_adam(jabas_dynhp_t* h, const jabas_group_t* groups, int ngroups,
                          const jabas_adam_hp_t* hp, void* stream)
{
    if (!h || !groups || !hp) return fail(JABAS_EINVAL, "null argument");
    if (ngroups < 1 || ngroups > JABAS_MAX_GROUPS) return fail(JABAS_EINVAL, "ngroups must be in [1, JABAS_MAX_GROUPS]");
    UpdHp v;
    int rc = jb_fill_adam_hp(v, groups, ngroups, hp);
    return rc ? rc : dynhp_push(h, v, OPT_ADAM, stream);
}

int jabas_dot_norms_f32(jabas_ctx_t* ctx, const float* a, const float* b, uint64_t n, double* stat3,
                        void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!a || !b || !stat3) return fail(JABAS_EINVAL, "a, b or stat3 is null");
    if (n == 0) return JABAS_OK;
    StatWs ws;
    if ((rc = ws_for(ctx, stream, &ws))) return rc;
    const int vec = (aligned16(a) && aligned16(b)) ? 1 : 0;
    int grid = 0;
    if ((rc = grid_for(ctx, dot_norms_kernel<false>, vec ? (n + 3) / 4 : n, vec ? kThreads * 4 : kThreads, &grid))) return rc;
    dot_norms_kernel<false><<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a, b, n, vec, ws, stat3);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_sumsq_f32(jabas_ctx_t* ctx, const float* x, uint64_t n, double* stat3, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!x || !stat3) return fail(JABAS_EINVAL, "x or stat3 is null");
    if (n == 0) return JABAS_OK;
    StatWs ws;
    if ((rc = ws_for(ctx, stream, &ws))) return rc;
    const int vec = aligned16(x) ? 1 : 0;
    int grid = 0;
    if ((rc = grid_for(ctx, dot_norms_kernel<true>, vec ? (n + 3) / 4 : n, vec ? kThreads * 4 : kThreads, &grid))) return rc;
    dot_norms_kernel<true><<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, x, n, vec, ws, stat3);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_clip_coef(jabas_ctx_t* ctx, const double* sumsq, double max_norm, float* coef_out, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!sumsq || !coef_out) return fail(JABAS_EINVAL, "sumsq or coef_out is null");
    if (!(max_norm > 0.0)) return fail(JABAS_EINVAL, "max_norm must be positive");
    clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, (float)max_norm, coef_out);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_cosine_finalize(jabas_ctx_t* ctx, const double* stat3, double eps, float* cos_out, void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!stat3 || !cos_out) return fail(JABAS_EINVAL, "stat3 or cos_out is null");
    cosine_finalize_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(stat3, eps, cos_out);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_replicate_f32(jabas_ctx_t* ctx, const float* src, float* const* dst, int ndst, uint64_t n,
                        void* stream)
{
    int rc = ctx_bind(ctx);
    if (rc) return rc;
    if (!src || (!dst && ndst > 0)) return fail(JABAS_EINVAL, "src or dst is null");
    if (ndst < 0 || ndst > JABAS_MAX_VSW) return fail(JABAS_EINVAL, "ndst must be in [0, JABAS_MAX_VSW]");
    RepArgs a;
    std::memset(&a, 0, sizeof(a));
    a.src = src; a.n = n; a.vec = aligned16(src) ? 1 : 0;
    for (int k = 0; k < ndst; ++k) {
        if (!dst[k]) return fail(JABAS_EINVAL, "dst[k] is null");
        if (dst[k] == src) continue;
        a.dst[a.ndst++] = dst[k];
        a.vec = a.vec && aligned16(dst[k]);
    }
    if (n == 0 || a.ndst == 0) return JABAS_OK;
    int grid = 0;
    if ((rc = grid_for(ctx, replicate_kernel, a.vec ? (n + 3) / 4 : n, a.vec ? kThreads * 4 : kThreads, &grid))) return rc;
    replicate_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

}  // extern "C"

// ----------------------------------------------------------------------------------
// jabas_dot_norms_static_f32: the dot/norms reduction for callers that must not allocate
// ----------------------------------------------------------------------------------
//
// Some hosts of this library cannot call cudaMalloc when the statistic is needed: code
// running inside a memory pool that owns the whole device (a training process whose
// caching allocator has reserved all HBM), a stream-ordered section that forbids
// synchronising allocations, or a plugin that is handed raw pointers and has no context
// of its own to keep a workspace in.  For them the per-CTA partial sums and the ticket
// counter live in this file-scope array instead of a workspace from cudaMalloc.  Every GPU
// that loads the library carries these 48 KiB + 256 B until the process exits.
constexpr int kStaticMaxCtas = 2048;     // partial-sum slots: 3 doubles per CTA
static __device__ __align__(256) unsigned char g_static_scratch[256 + sizeof(double) * 3 * kStaticMaxCtas];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char* g_static_ptr[kMaxDevices];   // device addresses of g_static_scratch, one per device
int g_static_sms[kMaxDevices];
}  // namespace

extern "C" int jabas_dot_norms_static_f32(const float* a, const float* b, uint64_t n, double* stat3,
                                          void* stream)
{
    if (!a || !b || !stat3) return fail(JABAS_EINVAL, "a, b or stat3 is null");
    if (n > JABAS_STATIC_MAX_ELEMS)
        return fail(JABAS_EINVAL, "n exceeds JABAS_STATIC_MAX_ELEMS (2^31 elements): split the input or "
                                  "use jabas_dot_norms_f32 with a context");
    if (n == 0) return JABAS_OK;
    int dev = -1;
    JB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(JABAS_EINVAL, "device index beyond the static table");
    unsigned char* base = nullptr;
    int sms = 0;
    {
        // First call on this device: resolve the DEVICE address of the array.  In host code the
        // symbol's name is only a host-side handle, never a pointer a kernel may dereference.
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[dev]) {
            void* p = nullptr;
            JB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
            JB_CUDA(cudaDeviceGetAttribute(&g_static_sms[dev], cudaDevAttrMultiProcessorCount, dev));
            g_static_ptr[dev] = static_cast<unsigned char*>(p);
        }
        base = g_static_ptr[dev];
        sms = g_static_sms[dev];
    }
    StatWs ws;
    ws.counter = reinterpret_cast<unsigned int*>(base);
    ws.partials = reinterpret_cast<double*>(base + 256);
    const int vec = (aligned16(a) && aligned16(b)) ? 1 : 0;
    const unsigned long long items = vec ? (n + 3) / 4 : n;
    const unsigned long long per_cta = vec ? kThreads * 4 : kThreads;
    unsigned long long grid = (items + per_cta - 1) / per_cta;
    const unsigned long long cap = (unsigned long long)sms * kMaxCtasPerSm;
    if (grid > cap) grid = cap;
    if (grid > (unsigned long long)kStaticMaxCtas) grid = kStaticMaxCtas;   // the kernel strides over the rest
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left: the ticket must start at zero.
    JB_CUDA(cudaMemsetAsync(ws.counter, 0, sizeof(unsigned int), st));
    dot_norms_kernel<false><<<(int)grid, kThreads, 0, st>>>(a, b, n, vec, ws, stat3);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}
