// The gradient path of several GPUs as ONE persistent kernel per GPU and launch:
//
//   aggregate  the K VSW gradients of this GPU -> undivided local sum S_r   (HBM-bound)
//   reduce     this GPU's shard of  g = sum_r fl(S_r / T)  and of the two
//              halves E / O (even / odd ranks), read from every GPU's S over
//              NVLink peer mappings                                          (NVLink-bound)
//   update     fused SGD-momentum / Adam / AdamW on the whole range with the
//              gradient gathered from the owners' shards over NVLink, new
//              weights written to all replicas                               (HBM-bound)
//
// The flat range is cut into chunks; every chunk into `nranks` shards (shard r is reduced by
// rank r); every shard into Q pieces of kPieceElems elements.  A piece of one phase is one work
// item.  Items stand in a queue ordered by pipeline step s = 0, 1, ...: step s holds the aggregate
// items of chunk s, the reduce items of chunk s-1 and the update items of chunk s-2, interleaved
// (one reduce item, then aggregate and update items in turn), so that at any moment the resident
// CTAs work on NVLink-bound and HBM-bound items together and the two resources overlap.  CTAs
// draw items with an atomic ticket, in queue order.
//
// Dependencies are flags, not collectives: when the Q aggregate pieces of (chunk, shard r) are
// done, this GPU stores the launch's epoch into rank r's flag block; a reduce item of rank r
// waits for the n flags of its chunk; when the Q reduce pieces of a chunk are done, rank r stores
// the epoch into every rank's flag block; an update item waits for the flag of the shard's
// owner.  An item only ever waits for items of the previous pipeline step, and tickets are drawn
// in order, so every item a wait depends on is already held by a running CTA on its GPU: no
// deadlock, whatever the number of resident CTAs.  Every wait is bounded by wall time; a wait that
// runs out records (phase, slot) in a status word, all CTAs of the launch drain, and the host
// reads the status — the kernel never traps and never spins for ever.
//
// Summation order is fixed (VSWs ascending, then ranks ascending, each term divided by T first:
// the reference's div_(T) before the SUM allreduce), so every rank computes bit-identical
// gradients and weights.  Plain peer loads and stores only: no multicast, no TMA.
#include "common.cuh"

#include <new>
#include <vector>

namespace jb_types {

constexpr int kExMaxRanks = 8;

struct ExArgs {
    const float* gk[JABAS_MAX_VSW];     // K local VSW gradient buffers (element 0 = element 0 of the flat buffer)
    float* w[JABAS_MAX_VSW];            // weight replicas written by the update (w[0] is read)
    float* m;
    float* v;
    const float* px[kExMaxRanks];       // every rank's undivided local sum, rank order (peer mappings)
    const float* pg[kExMaxRanks];       // every rank's reduced shards
    unsigned int* flags[kExMaxRanks];   // every rank's flag block
    float* px_local;
    float* pg_local;
    unsigned int* ctrl;                 // local: queue / done / launches / status, one 128-byte line each
    unsigned int* agg_cnt;              // local: [max_slots][kExMaxRanks] pieces done per (slot, shard)
    unsigned int* red_cnt;              // local: [max_slots]
    double* piece_stat;                 // local: [max_slots * Q][3]
    double* stat;                       // nullable: += this launch's (<E,O>, |E|^2, |O|^2) over this rank's shards
    const SegDev* segs;
    unsigned long long base, n;         // element range of the launch
    unsigned long long wait_ns;
    unsigned int chunk_elems, Q, nchunks, slot_base, max_slots;
    int nseg, K, Kw, nranks, rank;
    float divisor, half_divisor;
    const UpdHp* dyn;
    UpdHp hp;
};

}  // namespace jb_types

namespace {

constexpr unsigned kPieceElems = JABAS_EXCHANGE_PIECE;   // elements of one work item, per stream
constexpr int kExU = 2;                                  // 4-vectors per thread and inner step
constexpr unsigned kTileVecs = kThreads * kExU;

enum { CTL_QUEUE = 0, CTL_DONE = 32, CTL_LAUNCHES = 64, CTL_STATUS = 96, CTL_STAT_EPOCH = 128, CTL_WORDS = 160 };
enum { PH_AGG = 1, PH_RED = 2, PH_UPD = 3, PH_STAT = 4 };

__host__ __device__ inline size_t flag_words(unsigned max_slots) { return (size_t)max_slots * 2 * kExMaxRanks + 8 * kExMaxRanks; }
__device__ __forceinline__ unsigned agg_flag_idx(unsigned slot, int src) { return slot * kExMaxRanks + src; }
__device__ __forceinline__ unsigned red_flag_idx(unsigned max_slots, unsigned slot, int src)
{
    return (max_slots + slot) * kExMaxRanks + src;
}
__device__ __forceinline__ unsigned stat_idx(unsigned max_slots, int src) { return (2 * max_slots + src) * kExMaxRanks; }

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile(const unsigned* p)
{
    return *reinterpret_cast<const volatile unsigned*>(p);
}

// true once *f has reached `epoch`; false when `limit_ns` of wall time passed first (or another
// CTA of the launch already gave up).  The poll count is capped as well, so the loop ends even
// if the timer stood still.
__device__ __forceinline__ bool wait_epoch(const unsigned* f, unsigned epoch, unsigned long long limit_ns,
                                           const unsigned* status)
{
    if ((int)(ld_acquire_sys(f) - epoch) >= 0) return true;
    const unsigned long long t0 = gtime_ns();
    const unsigned long long max_polls = limit_ns / 64 + 4096;
    for (unsigned long long polls = 0; polls < max_polls; polls += 8) {
#pragma unroll 1
        for (int i = 0; i < 8; ++i) {
            if ((int)(ld_acquire_sys(f) - epoch) >= 0) return true;
            __nanosleep(40);
        }
        if (gtime_ns() - t0 > limit_ns) return false;
        if (ld_volatile(status) != 0u) return false;
    }
    return false;
}

__device__ __forceinline__ void record_timeout(const ExArgs& a, int phase, unsigned slot)
{
    atomicCAS(a.ctrl + CTL_STATUS, 0u, 0x80000000u | ((unsigned)phase << 24) | (slot & 0xffffffu));
}

// ---- aggregate piece: S = g_0 + ... + g_{K-1}, ascending k, undivided ---------------------
template <int KA>
__device__ __forceinline__ void agg_piece(const ExArgs& a, unsigned long long lo, unsigned long long hi)
{
    // eight gradient streams leave registers for one 4-vector per thread and step only
    constexpr int UA = KA > 4 ? 1 : kExU;
    const unsigned long long nvec = (hi - lo) >> 2;
    for (unsigned long long t0 = 0; t0 < nvec; t0 += (unsigned long long)kThreads * UA) {
        if (KA > 0) {
            float4 x[UA][KA > 0 ? KA : 1];
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (v < nvec) {
#pragma unroll
                    for (int k = 0; k < KA; ++k) x[u][k] = ld4(a.gk[k] + lo + 4 * v);
                }
            }
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (v < nvec) {
                    float4 s = x[u][0];
#pragma unroll
                    for (int k = 1; k < KA; ++k) s = add4(s, x[u][k]);
                    st4(a.px_local + lo + 4 * v, s);
                }
            }
        } else {
            float4 s[UA];
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (v < nvec) s[u] = ld4(a.gk[0] + lo + 4 * v);
            }
            for (int k = 1; k < a.K; ++k) {
#pragma unroll
                for (int u = 0; u < UA; ++u) {
                    const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                    if (v < nvec) s[u] = add4(s[u], ld4(a.gk[k] + lo + 4 * v));
                }
            }
#pragma unroll
            for (int u = 0; u < UA; ++u) {
                const unsigned long long v = t0 + (unsigned long long)u * kThreads + threadIdx.x;
                if (v < nvec) st4(a.px_local + lo + 4 * v, s[u]);
            }
        }
    }
}

// ---- reduce piece: g = sum_r fl(S_r / T) in rank order; E / O = even / odd ranks ----------
template <int NR>
__device__ __forceinline__ void red_piece(const ExArgs& a, unsigned long long lo, unsigned long long hi, Acc3& acc)
{
    const int n = NR > 0 ? NR : a.nranks;
    const unsigned long long nvec = (hi - lo) >> 2;
    const bool stat = a.stat != nullptr;
    for (unsigned long long v = threadIdx.x; v < nvec; v += kThreads) {
        const unsigned long long off = lo + 4 * v;
        float4 g, e, o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (NR > 0) {
            float4 x[NR > 0 ? NR : 1];
#pragma unroll
            for (int r = 0; r < NR; ++r) x[r] = ld4(a.px[r] + off);
            e = x[0];
            g = div4(x[0], a.divisor);
#pragma unroll
            for (int r = 1; r < NR; ++r) {
                g = add4(g, div4(x[r], a.divisor));
                if (r == 1) o = x[1]; else if (r & 1) o = add4(o, x[r]); else e = add4(e, x[r]);
            }
        } else {
            const float4 x0 = ld4(a.px[0] + off);
            e = x0;
            g = div4(x0, a.divisor);
            for (int r = 1; r < n; ++r) {
                const float4 y = ld4(a.px[r] + off);
                g = add4(g, div4(y, a.divisor));
                if (r == 1) o = y; else if (r & 1) o = add4(o, y); else e = add4(e, y);
            }
        }
        st4(a.pg_local + off, g);
        if (stat) acc_vec(acc, div4(e, a.half_divisor), div4(o, a.half_divisor));
    }
}

// ---- update piece: gradient from the owner's shard, fused optimizer step, K stores --------
template <int OPT>
__device__ __forceinline__ void upd_piece(const ExArgs& a, const UpdHp& H, const float* gsrc,
                                          unsigned long long lo, unsigned long long hi)
{
    const unsigned long long nvec = (hi - lo) >> 2;
    const bool use_m = OPT == OPT_ADAM || (H.flags & F_MOMENTUM);
    const bool load_m = OPT == OPT_ADAM || ((H.flags & F_MOMENTUM) && !(H.flags & F_FIRST));
    for (unsigned long long t0 = 0; t0 < nvec; t0 += kTileVecs) {
        float4 g[kExU], p[kExU], m[kExU], v[kExU];
#pragma unroll
        for (int u = 0; u < kExU; ++u) {
            const unsigned long long x = t0 + (unsigned long long)u * kThreads + threadIdx.x;
            m[u] = v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (x < nvec) {
                const unsigned long long off = lo + 4 * x;
                g[u] = ld4(gsrc + off);
                p[u] = ld4(a.w[0] + off);
                if (load_m) m[u] = ld4(a.m + off);
                if (OPT == OPT_ADAM) v[u] = ld4(a.v + off);
            }
        }
        // segment of the tile's first element, uniform over the CTA, looked up under the loads
        int seg0 = 0, gi0 = 0;
        bool uniform = true;
        if (a.segs) {
            const unsigned long long e0 = lo + 4 * t0;
            unsigned long long e1 = e0 + 4ull * kTileVecs;
            if (e1 > hi) e1 = hi;
            seg0 = seg_find(a.segs, a.nseg, e0);
            uniform = __ldg(&a.segs[seg0].end) >= e1;
            gi0 = (int)__ldg(&a.segs[seg0].group);
        }
#pragma unroll
        for (int u = 0; u < kExU; ++u) {
            const unsigned long long x = t0 + (unsigned long long)u * kThreads + threadIdx.x;
            if (x >= nvec) continue;
            const unsigned long long off = lo + 4 * x;
            if (uniform) {
                upd_math4<OPT>(H, H.grp[gi0], (H.wd_mask >> gi0) & 1u, g[u], p[u], m[u], v[u]);
            } else {
                int s = seg0;
                auto one = [&](int c, float gx, float& px, float& mx, float& vx) {
                    while (__ldg(&a.segs[s].end) <= off + c) ++s;
                    const int gi = (int)__ldg(&a.segs[s].group);
                    upd_math<OPT>(H, H.grp[gi], (H.wd_mask >> gi) & 1u, gx, px, mx, vx);
                };
                one(0, g[u].x, p[u].x, m[u].x, v[u].x);
                one(1, g[u].y, p[u].y, m[u].y, v[u].y);
                one(2, g[u].z, p[u].z, m[u].z, v[u].z);
                one(3, g[u].w, p[u].w, m[u].w, v[u].w);
            }
            for (int k = 0; k < a.Kw; ++k) st4(a.w[k] + off, p[u]);
            if (use_m) st4(a.m + off, m[u]);
            if (OPT == OPT_ADAM) st4(a.v + off, v[u]);
        }
    }
}

// One rank's share of a launch.  `ncta` CTAs of the grid (blockIdx.x) serve this rank.
template <int OPT, int KA, int NR>
__device__ __forceinline__ void exchange_body(const ExArgs& a, unsigned ncta)
{
    __shared__ UpdHp H;
    __shared__ unsigned s_ticket;
    __shared__ double s_red[3][kWarps];
    const int n = NR > 0 ? NR : a.nranks;
    if (a.dyn) {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(a.dyn);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&H);
        for (unsigned int i = threadIdx.x; i < sizeof(UpdHp) / 4; i += blockDim.x) dst[i] = __ldg(src + i);
    } else if (threadIdx.x == 0) {
        H = a.hp;
    }
    // Every CTA reads the launch counter before it draws its first ticket; the counter moves only
    // when the last CTA of the launch leaves, i.e. after every CTA has read it.
    const unsigned epoch = ld_volatile(a.ctrl + CTL_LAUNCHES) + 1u;
    const unsigned group_items = 2u * (unsigned)n + 1u;
    const unsigned step_items = a.Q * group_items;
    const unsigned total = (a.nchunks + 2u) * step_items;
    const unsigned long long end = a.base + a.n;
    const unsigned* status = a.ctrl + CTL_STATUS;
    unsigned* flags_local = a.flags[a.rank];
    if (threadIdx.x == 0) s_ticket = atomicAdd(a.ctrl + CTL_QUEUE, 1u);
    __syncthreads();
    unsigned t = s_ticket;
    while (t < total) {
        __syncthreads();                                  // s_ticket has been read by every thread
        unsigned nxt = 0;
        if (threadIdx.x == 0) nxt = atomicAdd(a.ctrl + CTL_QUEUE, 1u);   // in flight while this item runs
        const unsigned step = t / step_items, j = t % step_items;
        const unsigned grp = j / group_items, i = j % group_items;
        int phase;
        unsigned piece;                                   // piece index inside the chunk
        long long c;
        if (i == 0) { phase = PH_RED; c = (long long)step - 1; piece = (unsigned)a.rank * a.Q + grp; }
        else {
            const unsigned tt = i - 1u;
            piece = grp * (unsigned)n + (tt >> 1);
            if (tt & 1u) { phase = PH_UPD; c = (long long)step - 2; } else { phase = PH_AGG; c = (long long)step; }
        }
        bool ok = true;
        if (c >= 0 && c < (long long)a.nchunks) {
            const unsigned slot = a.slot_base + (unsigned)c;
            const int owner = (int)(piece / a.Q);
            unsigned long long lo = a.base + (unsigned long long)c * a.chunk_elems + (unsigned long long)piece * kPieceElems;
            unsigned long long hi = lo + kPieceElems;
            if (lo > end) lo = end;
            if (hi > end) hi = end;
            if (phase == PH_AGG) {
                agg_piece<KA>(a, lo, hi);
                __syncthreads();
                if (threadIdx.x == 0) {
                    __threadfence_system();
                    unsigned* cnt = a.agg_cnt + slot * kExMaxRanks + owner;
                    if (atomicAdd(cnt, 1u) == a.Q - 1u) {          // last piece of (chunk, shard): tell the owner
                        *cnt = 0u;
                        __threadfence_system();
                        st_release_sys(a.flags[owner] + agg_flag_idx(slot, a.rank), epoch);
                    }
                }
            } else if (phase == PH_RED) {
                if (threadIdx.x < n)
                    ok = wait_epoch(flags_local + agg_flag_idx(slot, threadIdx.x), epoch, a.wait_ns, status);
                ok = __syncthreads_and(ok);
                Acc3 acc = {0.0, 0.0, 0.0};
                if (ok) red_piece<NR>(a, lo, hi, acc);
                else if (threadIdx.x == 0) record_timeout(a, PH_RED, slot);
                if (a.stat) {
                    const Acc3 r = block_sum(acc, s_red);
                    if (threadIdx.x == 0) {
                        double* ps = a.piece_stat + 3ull * ((unsigned long long)slot * a.Q + grp);
                        ps[0] = r.d; ps[1] = r.a; ps[2] = r.b;
                    }
                }
                __syncthreads();
                if (ok && threadIdx.x == 0) {
                    __threadfence_system();
                    unsigned* cnt = a.red_cnt + slot;
                    if (atomicAdd(cnt, 1u) == a.Q - 1u) {          // this rank's shard of the chunk is reduced
                        *cnt = 0u;
                        __threadfence_system();
                        for (int r = 0; r < n; ++r)
                            st_release_sys(a.flags[r] + red_flag_idx(a.max_slots, slot, a.rank), epoch);
                    }
                }
            } else {
                if (threadIdx.x == 0)
                    ok = wait_epoch(flags_local + red_flag_idx(a.max_slots, slot, owner), epoch, a.wait_ns, status);
                ok = __syncthreads_and(ok);
                if (ok) {
                    upd_piece<OPT>(a, H, a.pg[owner], lo, hi);
                } else if (threadIdx.x == 0) {
                    record_timeout(a, PH_UPD, slot);
                }
            }
        }
        if (threadIdx.x == 0) s_ticket = (!ok || ld_volatile(status) != 0u) ? 0xffffffffu : nxt;
        __syncthreads();
        t = s_ticket;
    }
    // the last CTA to leave adds this launch's piece sums in slot order, rewinds the queue and
    // advances the launch counter
    __shared__ int is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = atomicAdd(a.ctrl + CTL_DONE, 1u) == ncta - 1u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (a.stat) {
        Acc3 s = {0.0, 0.0, 0.0};
        const unsigned long long first = (unsigned long long)a.slot_base * a.Q;
        const unsigned long long cnt = (unsigned long long)a.nchunks * a.Q;
        if (ld_volatile(status) == 0u) {
            for (unsigned long long q = threadIdx.x; q < cnt; q += kThreads) {
                s.d += __ldcg(a.piece_stat + 3 * (first + q) + 0);
                s.a += __ldcg(a.piece_stat + 3 * (first + q) + 1);
                s.b += __ldcg(a.piece_stat + 3 * (first + q) + 2);
            }
        }
        s = block_sum(s, s_red);
        if (threadIdx.x == 0) { a.stat[0] += s.d; a.stat[1] += s.a; a.stat[2] += s.b; }
    }
    if (threadIdx.x == 0) {
        a.ctrl[CTL_QUEUE] = 0u;
        a.ctrl[CTL_DONE] = 0u;
        a.ctrl[CTL_LAUNCHES] = epoch;
    }
}

// Two CTAs per SM: the update item keeps two tiles of four streams in registers.
template <int OPT, int KA, int NR>
__global__ void __launch_bounds__(kThreads, 2) exchange_kernel(const ExArgs a)
{
    exchange_body<OPT, KA, NR>(a, gridDim.x);
}

// Several ranks' exchanges in ONE launch on ONE GPU (blockIdx.y = rank): kernels that wait on
// one another may not run as separate launches on a GPU, so single-GPU tests of the protocol
// use this form, with the grid sized so that every CTA is resident.
template <int OPT, int KA, int NR>
__global__ void __launch_bounds__(kThreads, 2) exchange_emu_kernel(const ExArgs* ranks)
{
    __shared__ ExArgs a;
    {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(ranks + blockIdx.y);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&a);
        for (unsigned int i = threadIdx.x; i < sizeof(ExArgs) / 4; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
    exchange_body<OPT, KA, NR>(a, gridDim.x);
}

// ---- statistic across ranks: publish, wait, sum in rank order, finalize ---------------------
struct ExStatArgs {
    unsigned int* flags[kExMaxRanks];
    unsigned int* ctrl;
    double* stat;            // in: this rank's sums; out: the sums over all ranks
    float* cos_out;
    unsigned long long wait_ns;
    double eps;
    unsigned int max_slots;
    int nranks, rank;
};

__device__ __forceinline__ void exchange_cosine_body(const ExStatArgs& a)
{
    const unsigned epoch = ld_volatile(a.ctrl + CTL_STAT_EPOCH) + 1u;
    if (threadIdx.x == 0) {
        const double s0 = a.stat[0], s1 = a.stat[1], s2 = a.stat[2];
        for (int r = 0; r < a.nranks; ++r) {
            unsigned int* blk = a.flags[r] + stat_idx(a.max_slots, a.rank);
            double* d = reinterpret_cast<double*>(blk);
            d[0] = s0; d[1] = s1; d[2] = s2;
        }
        __threadfence_system();
        for (int r = 0; r < a.nranks; ++r)
            st_release_sys(a.flags[r] + stat_idx(a.max_slots, a.rank) + 6, epoch);
    }
    bool ok = true;
    if ((int)threadIdx.x < a.nranks)
        ok = wait_epoch(a.flags[a.rank] + stat_idx(a.max_slots, threadIdx.x) + 6, epoch, a.wait_ns,
                        a.ctrl + CTL_STATUS);
    ok = __syncthreads_and(ok);
    if (threadIdx.x == 0) {
        if (ok) {
            double t0 = 0.0, t1 = 0.0, t2 = 0.0;
            for (int r = 0; r < a.nranks; ++r) {
                const double* d = reinterpret_cast<const double*>(a.flags[a.rank] + stat_idx(a.max_slots, r));
                t0 += __ldcg(d + 0); t1 += __ldcg(d + 1); t2 += __ldcg(d + 2);
            }
            a.stat[0] = t0; a.stat[1] = t1; a.stat[2] = t2;
            double den = t1 * t2;
            if (den < a.eps * a.eps) den = a.eps * a.eps;
            a.cos_out[0] = (float)(t0 / sqrt(den));
        } else {
            atomicCAS(a.ctrl + CTL_STATUS, 0u, 0x80000000u | ((unsigned)PH_STAT << 24));
        }
        a.ctrl[CTL_STAT_EPOCH] = epoch;
    }
}

__global__ void __launch_bounds__(32) exchange_cosine_kernel(const ExStatArgs a) { exchange_cosine_body(a); }

__global__ void __launch_bounds__(32) exchange_cosine_emu_kernel(const ExStatArgs* ranks)
{
    __shared__ ExStatArgs a;
    {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(ranks + blockIdx.x);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&a);
        for (unsigned int i = threadIdx.x; i < sizeof(ExStatArgs) / 4; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
    exchange_cosine_body(a);
}

}  // namespace

struct jabas_exchange {
    jabas_ctx_t* ctx = nullptr;
    int nranks = 0, rank = 0;
    unsigned max_slots = 0, Q = 0;
    const float* px[kExMaxRanks] = {};
    const float* pg[kExMaxRanks] = {};
    unsigned int* flags[kExMaxRanks] = {};
    unsigned int* d_local = nullptr;     // ctrl | agg_cnt | red_cnt | piece_stat
    size_t local_bytes = 0;
    ExArgs* d_emu = nullptr;             // argument blocks of the single-GPU multi-rank form
    int occ = 0;
};

namespace {

typedef void (*ExKernel)(const ExArgs);
typedef void (*ExEmuKernel)(const ExArgs*);

template <int OPT, int KA, int NR>
void pick(ExKernel* k, ExEmuKernel* e)
{
    *k = exchange_kernel<OPT, KA, NR>;
    *e = exchange_emu_kernel<OPT, KA, NR>;
}

template <int OPT, int KA>
void pick_nr(int n, ExKernel* k, ExEmuKernel* e)
{
    switch (n) {
    case 2: pick<OPT, KA, 2>(k, e); break;
    case 4: pick<OPT, KA, 4>(k, e); break;
    case 8: pick<OPT, KA, 8>(k, e); break;
    default: pick<OPT, KA, 0>(k, e); break;
    }
}

template <int OPT>
void pick_ka(int K, int n, ExKernel* k, ExEmuKernel* e)
{
    switch (K) {
    case 1: pick_nr<OPT, 1>(n, k, e); break;
    case 2: pick_nr<OPT, 2>(n, k, e); break;
    case 4: pick_nr<OPT, 4>(n, k, e); break;
    case 8: pick_nr<OPT, 8>(n, k, e); break;
    default: pick_nr<OPT, 0>(n, k, e); break;
    }
}

}  // namespace

extern "C" {

size_t jabas_exchange_flag_words(uint32_t max_slots) { return flag_words(max_slots); }

int jabas_exchange_create(jabas_ctx_t* ctx, const jabas_exchange_desc_t* d, jabas_exchange_t** out)
{
    int rc = jb_ctx_bind(ctx);
    if (rc) return rc;
    if (!d || !out) return fail(JABAS_EINVAL, "exchange: null argument");
    *out = nullptr;
    if (d->nranks < 2 || d->nranks > kExMaxRanks) return fail(JABAS_EINVAL, "exchange: 2..8 ranks");
    if (d->rank < 0 || d->rank >= d->nranks) return fail(JABAS_EINVAL, "exchange: rank out of range");
    if (d->max_slots < 1 || d->max_slots > (1u << 20)) return fail(JABAS_EINVAL, "exchange: max_slots out of range");
    if (d->pieces_per_shard < 1 || d->pieces_per_shard > 4096)
        return fail(JABAS_EINVAL, "exchange: pieces_per_shard must be in [1, 4096]");
    if (!d->px || !d->pg || !d->flags) return fail(JABAS_EINVAL, "exchange: null buffer table");
    jabas_exchange_t* ex = new (std::nothrow) jabas_exchange_t();
    if (!ex) return fail(JABAS_ENOMEM, "out of host memory");
    ex->ctx = ctx; ex->nranks = d->nranks; ex->rank = d->rank; ex->max_slots = d->max_slots;
    ex->Q = d->pieces_per_shard;
    for (int r = 0; r < d->nranks; ++r) {
        if (!d->px[r] || !d->pg[r] || !d->flags[r] || !aligned16(d->px[r]) || !aligned16(d->pg[r]) ||
            !aligned16(d->flags[r])) {
            delete ex;
            return fail(JABAS_EINVAL, "exchange: buffers must be non-null and 16-byte aligned");
        }
        ex->px[r] = d->px[r]; ex->pg[r] = d->pg[r]; ex->flags[r] = d->flags[r];
    }
    const size_t words = CTL_WORDS + (size_t)ex->max_slots * kExMaxRanks + ex->max_slots;
    const size_t stat_off = (words * 4 + 255) / 256 * 256;
    ex->local_bytes = stat_off + sizeof(double) * 3 * (size_t)ex->max_slots * ex->Q;
    cudaError_t e = cudaMalloc(&ex->d_local, ex->local_bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->d_local, 0, ex->local_bytes);
    if (e != cudaSuccess) {
        if (ex->d_local) cudaFree(ex->d_local);
        delete ex;
        return fail(JABAS_ECUDA, cudaGetErrorString(e));
    }
    *out = ex;
    return JABAS_OK;
}

int jabas_exchange_destroy(jabas_exchange_t* ex)
{
    if (!ex) return JABAS_OK;
    int rc = jb_ctx_bind(ex->ctx);
    if (rc == JABAS_OK) {
        cudaFree(ex->d_local);
        if (ex->d_emu) cudaFree(ex->d_emu);
    }
    delete ex;
    return rc;
}

int jabas_exchange_reset(jabas_exchange_t* ex)
{
    if (!ex) return fail(JABAS_EINVAL, "exchange is null");
    int rc = jb_ctx_bind(ex->ctx);
    if (rc) return rc;
    JB_CUDA(cudaDeviceSynchronize());
    JB_CUDA(cudaMemset(ex->d_local, 0, ex->local_bytes));
    return JABAS_OK;
}

int jabas_exchange_status(jabas_exchange_t* ex, uint32_t* status, uint32_t* launches)
{
    if (!ex || !status) return fail(JABAS_EINVAL, "exchange or status is null");
    int rc = jb_ctx_bind(ex->ctx);
    if (rc) return rc;
    unsigned int h[CTL_WORDS];
    JB_CUDA(cudaMemcpy(h, ex->d_local, sizeof(h), cudaMemcpyDeviceToHost));
    *status = h[CTL_STATUS];
    if (launches) *launches = h[CTL_LAUNCHES];
    return JABAS_OK;
}

static int fill_args(jabas_exchange_t* ex, const jabas_exchange_bufs_t& b, ExArgs& a, uint64_t n, uint64_t base,
                     uint32_t slot_base, float divisor, float half_divisor, const jabas_layout_t* layout,
                     const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* sgd,
                     const jabas_adam_hp_t* adam)
{
    jabas_ctx_t* ctx = ex->ctx;
    std::memset(&a, 0, sizeof(a));
    if (!b.grads || !b.w) return fail(JABAS_EINVAL, "exchange: grads or w is null");
    if (b.Kg < 1 || b.Kg > JABAS_MAX_VSW || b.K < 1 || b.K > JABAS_MAX_VSW)
        return fail(JABAS_EINVAL, "exchange: K must be in [1, JABAS_MAX_VSW]");
    if ((n & 3ull) || (base & 3ull)) return fail(JABAS_EINVAL, "exchange: base and n must be multiples of 4 elements");
    if (!(divisor != 0.0f)) return fail(JABAS_EINVAL, "divisor must be non-zero");
    if (b.stat3 && !(half_divisor != 0.0f)) return fail(JABAS_EINVAL, "half_divisor must be non-zero");
    if (b.stat3 && (ex->nranks & 1)) return fail(JABAS_EINVAL, "the two-half statistic needs an even number of ranks");
    if (!groups || ngroups < 1 || ngroups > JABAS_MAX_GROUPS)
        return fail(JABAS_EINVAL, "ngroups must be in [1, JABAS_MAX_GROUPS]");
    if ((sgd == nullptr) == (adam == nullptr)) return fail(JABAS_EINVAL, "exchange: give exactly one of sgd / adam");
    for (int k = 0; k < b.Kg; ++k) {
        if (!b.grads[k] || !aligned16(b.grads[k])) return fail(JABAS_EINVAL, "exchange: grads[k] null or not 16-byte aligned");
        a.gk[k] = b.grads[k];
    }
    for (int k = 0; k < b.K; ++k) {
        if (!b.w[k] || !aligned16(b.w[k])) return fail(JABAS_EINVAL, "exchange: w[k] null or not 16-byte aligned");
        a.w[k] = b.w[k];
    }
    if ((b.m && !aligned16(b.m)) || (b.v && !aligned16(b.v))) return fail(JABAS_EINVAL, "exchange: m / v not 16-byte aligned");
    a.m = b.m; a.v = b.v; a.stat = b.stat3;
    for (int r = 0; r < ex->nranks; ++r) { a.px[r] = ex->px[r]; a.pg[r] = ex->pg[r]; a.flags[r] = ex->flags[r]; }
    a.px_local = const_cast<float*>(ex->px[ex->rank]);
    a.pg_local = const_cast<float*>(ex->pg[ex->rank]);
    a.ctrl = ex->d_local;
    a.agg_cnt = ex->d_local + CTL_WORDS;
    a.red_cnt = a.agg_cnt + (size_t)ex->max_slots * kExMaxRanks;
    const size_t words = CTL_WORDS + (size_t)ex->max_slots * kExMaxRanks + ex->max_slots;
    a.piece_stat = reinterpret_cast<double*>(reinterpret_cast<char*>(ex->d_local) + (words * 4 + 255) / 256 * 256);
    a.base = base; a.n = n;
    a.wait_ns = (unsigned long long)(ctx->peer_wait_ms * 1e6);
    a.Q = ex->Q;
    const unsigned long long chunk = (unsigned long long)ex->nranks * ex->Q * kPieceElems;
    if (chunk > 0xffffffffull) return fail(JABAS_EINVAL, "exchange: chunk too large");
    a.chunk_elems = (unsigned)chunk;
    const unsigned long long nchunks = (n + chunk - 1) / chunk;
    if ((unsigned long long)slot_base + nchunks > ex->max_slots)
        return fail(JABAS_EINVAL, "exchange: the range needs more flag slots than the exchange was created with");
    if ((nchunks + 2) * (unsigned long long)ex->Q * (2ull * ex->nranks + 1) >= 0xfffffff0ull)
        return fail(JABAS_EINVAL, "exchange: too many work items for one launch");
    a.nchunks = (unsigned)nchunks; a.slot_base = slot_base; a.max_slots = ex->max_slots;
    a.K = b.Kg; a.Kw = b.K; a.nranks = ex->nranks; a.rank = ex->rank;
    a.divisor = divisor; a.half_divisor = half_divisor;
    if (layout) {
        if (layout->device != ctx->device) return fail(JABAS_EINVAL, "layout belongs to another device");
        if (base + n > layout->total) return fail(JABAS_EINVAL, "base + n exceeds the layout");
        if (layout->max_group >= ngroups)
            return fail(JABAS_EINVAL, "the layout names a param group that the call does not provide");
        a.segs = layout->dsegs; a.nseg = layout->nseg;
    }
    int rc;
    if (sgd) {
        if (sgd->momentum != 0.0 && !b.m) return fail(JABAS_EINVAL, "momentum != 0 needs a momentum buffer");
        if (sgd->nesterov && (sgd->momentum <= 0.0 || sgd->dampening != 0.0))
            return fail(JABAS_EINVAL, "nesterov needs momentum > 0 and dampening == 0");
        if (sgd->grad_scale || sgd->peer_grad) return fail(JABAS_EINVAL, "exchange: grad_scale / peer_grad are not supported");
        if ((rc = jb_fill_sgd_hp(a.hp, groups, ngroups, sgd))) return rc;
        if (sgd->dynamic) {
            if (sgd->dynamic->kind != OPT_SGD) return fail(JABAS_EINVAL, "the dynamic block holds Adam hyper-parameters");
            a.dyn = sgd->dynamic->dev;
        }
    } else {
        if (!b.m || !b.v) return fail(JABAS_EINVAL, "exp_avg and exp_avg_sq buffers are required");
        if (adam->grad_scale || adam->peer_grad) return fail(JABAS_EINVAL, "exchange: grad_scale / peer_grad are not supported");
        if ((rc = jb_fill_adam_hp(a.hp, groups, ngroups, adam))) return rc;
        if (adam->dynamic) {
            if (adam->dynamic->kind != OPT_ADAM) return fail(JABAS_EINVAL, "the dynamic block holds SGD hyper-parameters");
            a.dyn = adam->dynamic->dev;
        }
    }
    return JABAS_OK;
}

int jabas_exchange_step_f32(jabas_exchange_t* const* exs, const jabas_exchange_bufs_t* bufs, int nlocal,
                            uint64_t n, uint64_t base, uint32_t slot_base, float divisor, float half_divisor,
                            const jabas_layout_t* layout, const jabas_group_t* groups, int ngroups,
                            const jabas_sgd_hp_t* sgd, const jabas_adam_hp_t* adam, void* stream)
{
    if (!exs || !bufs || nlocal < 1 || !exs[0]) return fail(JABAS_EINVAL, "exchange: null argument");
    jabas_exchange_t* ex0 = exs[0];
    if (nlocal != 1 && nlocal != ex0->nranks)
        return fail(JABAS_EINVAL, "exchange: nlocal is 1 (one rank per GPU) or the number of ranks (all ranks on one GPU)");
    int rc = jb_ctx_bind(ex0->ctx);
    if (rc) return rc;
    if (n == 0) return JABAS_OK;
    ExKernel kern = nullptr;
    ExEmuKernel emu = nullptr;
    if (sgd) pick_ka<OPT_SGD>(bufs[0].Kg, ex0->nranks, &kern, &emu);
    else pick_ka<OPT_ADAM>(bufs[0].Kg, ex0->nranks, &kern, &emu);
    jabas_ctx_t* ctx = ex0->ctx;
    int per_sm = 0;
    {
        const void* key = nlocal == 1 ? reinterpret_cast<const void*>(kern) : reinterpret_cast<const void*>(emu);
        std::lock_guard<std::mutex> lk(ctx->mu);
        auto it = ctx->occ.find(key);
        if (it != ctx->occ.end()) per_sm = it->second;
        if (per_sm == 0) {
            cudaError_t e = nlocal == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, 0)
                                        : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, emu, kThreads, 0);
            if (e != cudaSuccess) return fail(JABAS_ECUDA, cudaGetErrorString(e));
            if (per_sm < 1) per_sm = 1;
            if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
            ctx->occ[key] = per_sm;
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (nlocal == 1) {
        ExArgs a;
        if ((rc = fill_args(ex0, bufs[0], a, n, base, slot_base, divisor, half_divisor, layout, groups, ngroups, sgd, adam)))
            return rc;
        const unsigned long long items = (unsigned long long)(a.nchunks + 2) * a.Q * (2ull * a.nranks + 1);
        unsigned long long grid = (unsigned long long)ctx->sm_count * per_sm;
        if (grid > items) grid = items;
        kern<<<(unsigned)grid, kThreads, 0, st>>>(a);
        JB_CUDA(cudaGetLastError());
        return JABAS_OK;
    }
    // all ranks on this GPU, one launch: every CTA must be resident, because ranks wait on one another
    std::vector<ExArgs> h((size_t)nlocal);
    for (int r = 0; r < nlocal; ++r) {
        if (!exs[r] || exs[r]->ctx != ctx || exs[r]->nranks != nlocal || exs[r]->rank != r)
            return fail(JABAS_EINVAL, "exchange: the single-GPU form takes the ranks 0..n-1 of one context, in order");
        if (bufs[r].Kg != bufs[0].Kg) return fail(JABAS_EINVAL, "exchange: every rank must have the same number of VSWs here");
        if ((rc = fill_args(exs[r], bufs[r], h[r], n, base, slot_base, divisor, half_divisor, layout, groups, ngroups, sgd, adam)))
            return rc;
    }
    if (!ex0->d_emu) JB_CUDA(cudaMalloc(&ex0->d_emu, sizeof(ExArgs) * kExMaxRanks));
    JB_CUDA(cudaMemcpyAsync(ex0->d_emu, h.data(), sizeof(ExArgs) * nlocal, cudaMemcpyHostToDevice, st));
    JB_CUDA(cudaStreamSynchronize(st));          // h leaves scope; this form is for tests
    unsigned gx = (unsigned)((ctx->sm_count * per_sm) / nlocal);
    if (gx < 1) return fail(JABAS_EINVAL, "exchange: the GPU cannot hold one CTA per rank");
    emu<<<dim3(gx, (unsigned)nlocal), kThreads, 0, st>>>(ex0->d_emu);
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

int jabas_exchange_cosine(jabas_exchange_t* const* exs, double* const* stat3, float* const* cos_out, int nlocal,
                          double eps, void* stream)
{
    if (!exs || !stat3 || !cos_out || nlocal < 1 || !exs[0]) return fail(JABAS_EINVAL, "exchange: null argument");
    jabas_exchange_t* ex0 = exs[0];
    if (nlocal != 1 && nlocal != ex0->nranks) return fail(JABAS_EINVAL, "exchange: nlocal is 1 or the number of ranks");
    int rc = jb_ctx_bind(ex0->ctx);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::vector<ExStatArgs> h((size_t)nlocal);
    for (int r = 0; r < nlocal; ++r) {
        jabas_exchange_t* ex = exs[r];
        if (!ex || !stat3[r] || !cos_out[r]) return fail(JABAS_EINVAL, "exchange: null argument");
        if (nlocal > 1 && (ex->ctx != ex0->ctx || ex->nranks != nlocal || ex->rank != r))
            return fail(JABAS_EINVAL, "exchange: the single-GPU form takes the ranks 0..n-1 of one context, in order");
        ExStatArgs& a = h[r];
        std::memset(&a, 0, sizeof(a));
        for (int j = 0; j < ex->nranks; ++j) a.flags[j] = ex->flags[j];
        a.ctrl = ex->d_local; a.stat = stat3[r]; a.cos_out = cos_out[r];
        a.wait_ns = (unsigned long long)(ex->ctx->peer_wait_ms * 1e6);
        a.eps = eps; a.max_slots = ex->max_slots; a.nranks = ex->nranks; a.rank = ex->rank;
    }
    if (nlocal == 1) {
        exchange_cosine_kernel<<<1, 32, 0, st>>>(h[0]);
    } else {
        static_assert(sizeof(ExStatArgs) <= sizeof(ExArgs), "the emulation block is sized for ExArgs");
        if (!ex0->d_emu) JB_CUDA(cudaMalloc(&ex0->d_emu, sizeof(ExArgs) * kExMaxRanks));
        JB_CUDA(cudaMemcpyAsync(ex0->d_emu, h.data(), sizeof(ExStatArgs) * nlocal, cudaMemcpyHostToDevice, st));
        JB_CUDA(cudaStreamSynchronize(st));
        exchange_cosine_emu_kernel<<<nlocal, 32, 0, st>>>(reinterpret_cast<const ExStatArgs*>(ex0->d_emu));
    }
    JB_CUDA(cudaGetLastError());
    return JABAS_OK;
}

}  // extern "C"
