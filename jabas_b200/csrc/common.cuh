// Device helpers, argument blocks and host-side objects shared by the translation units of
// libjabas_b200.so (gradpath.cu: the per-phase kernels; exchange.cu: the pipelined cross-GPU
// exchange).  Everything device-side is inline, so the files link without relocatable
// device code.
#pragma once

#include "jabas_b200.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

// Records the message jabas_last_error() returns for the calling thread; returns `code`.
int jb_fail(int code, const std::string& msg);

#define JB_CUDA(expr)                                                                        \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return jb_fail(JABAS_ECUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)

// Plain data shared between translation units (named namespace: one identity for the linker).
namespace jb_types {

struct Acc3 {
    double d, a, b;
};

struct StatWs {
    double* partials;       // 3 doubles per CTA
    unsigned int* counter;  // ticket, returns to 0 at the end of every launch
};

struct SegDev {
    unsigned long long begin, end;
    unsigned int group, pad;
};

struct GroupDev {
    float wd;      // weight decay
    float s0;      // SGD: -lr             Adam: 1 - lr*wd (decoupled decay factor)
    float s1;      // SGD: unused          Adam: -(lr / (1 - beta1^t))
    float s2;      // SGD: unused          Adam: sqrt(1 - beta2^t)
};

// Everything an update kernel needs that may change from one iteration to the next.
struct UpdHp {
    GroupDev grp[JABAS_MAX_GROUPS];
    unsigned int flags;
    unsigned int wd_mask;     // bit i: group i has weight_decay != 0
    float c0, c1, c2, c3, c4; // SGD: mu, 1-dampening | Adam: b1, b2, 1-b1, 1-b2, eps
    float pad;
};

enum { OPT_SGD = 0, OPT_ADAM = 1 };
enum { F_NESTEROV = 1, F_FIRST = 2, F_MOMENTUM = 4, F_DECOUPLED = 8 };

}  // namespace jb_types
using namespace jb_types;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxCtasPerSm = 8;

constexpr double kDefaultStagingWaitMs = 50.0;   // a 4 KB copy from local HBM takes microseconds
constexpr double kDefaultPeerWaitMs = 5000.0;    // waits on another GPU's progress absorb rank skew

inline int fail(int code, const std::string& msg) { return jb_fail(code, msg); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ----------------------------------------------------------------------------------
// device helpers
// ----------------------------------------------------------------------------------

// Plain (coherent) 128-bit load that does not allocate in L1: every input is read once
// per launch, and outputs may alias inputs, which rules out the non-coherent path.
__device__ __forceinline__ float4 ld4(const float* p)
{
    float4 v;
    asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st4(float* p, float4 v)
{
    *reinterpret_cast<float4*>(p) = v;
}

__device__ __forceinline__ unsigned long long gtime_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier and bulk-copy (TMA, untiled, no multicast) primitives ---------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p)
{
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* b, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* b, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* b, unsigned parity)
{
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(smem_u32(b)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// false: the copies of this stage did not land within `limit_ns` nanoseconds of wall time
// (the limit is a time, not a poll count, so it does not depend on how long one poll takes)
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* b, unsigned parity, unsigned long long limit_ns)
{
    if (mbar_try_wait(b, parity)) return true;
    const unsigned long long t0 = gtime_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(b, parity)) return true;
        if (gtime_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src, unsigned bytes, unsigned long long* b)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(b))
                 : "memory");
}
// orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* b)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}

__device__ __forceinline__ void acc_vec(Acc3& acc, float4 e, float4 o)
{
    float d = __fmul_rn(e.x, o.x), a = __fmul_rn(e.x, e.x), b = __fmul_rn(o.x, o.x);
    d = __fmaf_rn(e.y, o.y, d); a = __fmaf_rn(e.y, e.y, a); b = __fmaf_rn(o.y, o.y, b);
    d = __fmaf_rn(e.z, o.z, d); a = __fmaf_rn(e.z, e.z, a); b = __fmaf_rn(o.z, o.z, b);
    d = __fmaf_rn(e.w, o.w, d); a = __fmaf_rn(e.w, e.w, a); b = __fmaf_rn(o.w, o.w, b);
    acc.d += (double)d; acc.a += (double)a; acc.b += (double)b;
}
__device__ __forceinline__ void acc_one(Acc3& acc, float e, float o)
{
    acc.d += (double)e * (double)o; acc.a += (double)e * (double)e; acc.b += (double)o * (double)o;
}

__device__ __forceinline__ Acc3 warp_sum(Acc3 v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v.d += __shfl_down_sync(0xffffffffu, v.d, off);
        v.a += __shfl_down_sync(0xffffffffu, v.a, off);
        v.b += __shfl_down_sync(0xffffffffu, v.b, off);
    }
    return v;
}

// CTA-wide sum, valid in thread 0.
__device__ __forceinline__ Acc3 block_sum(Acc3 v, double (*sm)[kWarps])
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sm[0][warp] = v.d; sm[1][warp] = v.a; sm[2][warp] = v.b; }
    __syncthreads();
    Acc3 r = {0.0, 0.0, 0.0};
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { r.d += sm[0][w]; r.a += sm[1][w]; r.b += sm[2][w]; }
    }
    return r;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b)
{
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 div4(float4 a, float d)
{
    return make_float4(__fdiv_rn(a.x, d), __fdiv_rn(a.y, d), __fdiv_rn(a.z, d), __fdiv_rn(a.w, d));
}

// ----------------------------------------------------------------------------------
// optimizer update: hyper-parameter block, segment table, arithmetic
// ----------------------------------------------------------------------------------

// index of the segment that holds element `idx` (segments are contiguous and sorted)
__device__ __forceinline__ int seg_find(const SegDev* segs, int nseg, unsigned long long idx)
{
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(&segs[mid].end) <= idx) lo = mid + 1; else hi = mid;
    }
    return lo;
}

template <int OPT>
__device__ __forceinline__ void upd_math(const UpdHp& a, const GroupDev& h, bool has_wd, float g,
                                         float& p, float& m, float& v)
{
    if (OPT == OPT_SGD) {
        float d = g;
        if (has_wd) d = __fmaf_rn(h.wd, p, d);
        if (a.flags & F_MOMENTUM) {
            float b;
            if (a.flags & F_FIRST) b = d;
            else b = __fmaf_rn(a.c1, d, __fmul_rn(a.c0, m));
            m = b;
            d = (a.flags & F_NESTEROV) ? __fmaf_rn(a.c0, b, d) : b;
        }
        p = __fmaf_rn(h.s0, d, p);
    } else {
        if (a.flags & F_DECOUPLED) p = __fmul_rn(p, h.s0);
        else if (has_wd) g = __fmaf_rn(h.wd, p, g);
        m = __fmaf_rn(a.c2, g, __fmul_rn(a.c0, m));
        v = __fmaf_rn(__fmul_rn(a.c3, g), g, __fmul_rn(a.c1, v));
        const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), h.s2), a.c4);
        p = __fmaf_rn(h.s1, __fdiv_rn(m, denom), p);
    }
}

template <int OPT>
__device__ __forceinline__ void upd_math4(const UpdHp& a, const GroupDev& h, bool has_wd, float4 g,
                                          float4& p, float4& m, float4& v)
{
    upd_math<OPT>(a, h, has_wd, g.x, p.x, m.x, v.x);
    upd_math<OPT>(a, h, has_wd, g.y, p.y, m.y, v.y);
    upd_math<OPT>(a, h, has_wd, g.z, p.z, m.z, v.z);
    upd_math<OPT>(a, h, has_wd, g.w, p.w, m.w, v.w);
}

}  // namespace

// ----------------------------------------------------------------------------------
// host-side objects behind the opaque handles of the C ABI
// ----------------------------------------------------------------------------------

struct jabas_ctx {
    int device = 0;
    int sm_count = 0;
    int max_grid = 0;
    std::mutex mu;
    std::unordered_map<void*, StatWs> ws;   // one reduction workspace per stream
    std::unordered_map<const void*, int> occ;
    int staging = JABAS_STAGING_REGISTER;   // how the update kernels fetch their tiles
    unsigned int* d_timeouts = nullptr;     // bulk staging: waits that ran out (device counter)
    double staging_wait_ms = kDefaultStagingWaitMs;
    double peer_wait_ms = kDefaultPeerWaitMs;
    unsigned int stall_tx = 0;              // test seam, see jabas_ctx_inject_staging_stall
};

struct jabas_layout {
    int device = 0;
    int nseg = 0;
    int max_group = 0;
    unsigned long long total = 0;
    SegDev* dsegs = nullptr;
};

// Device-resident hyper-parameter block.  A captured CUDA graph bakes kernel arguments in;
// what changes every iteration (lr, Adam step, first-step flag) therefore lives in device
// memory and is refreshed by a small stream-ordered copy BEFORE each replay, outside the
// graph, from a ring of pinned slots (a slot is reused only after its copy has completed).
struct jabas_dynhp {
    static constexpr int kSlots = 8;
    int device = 0;
    int kind = -1;                  // OPT_SGD / OPT_ADAM once pushed
    UpdHp* dev = nullptr;
    UpdHp* pinned = nullptr;        // kSlots entries
    cudaEvent_t done[kSlots] = {};
    int next = 0;
    std::mutex mu;
};

// Makes the context's device current.
int jb_ctx_bind(jabas_ctx_t* ctx);
// Host -> kernel form of the hyper-parameters: fp64 scalars rounded to fp32 once.
int jb_fill_sgd_hp(UpdHp& h, const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* hp);
int jb_fill_adam_hp(UpdHp& h, const jabas_group_t* groups, int ngroups, const jabas_adam_hp_t* hp);
