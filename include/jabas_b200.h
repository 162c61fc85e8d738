/*
 * jabas_b200 — C ABI of the B200 (sm_100a) gradient-path library, libjabas_b200.so.
 *
 * The reference (unist-ssl/JABAS on top of IIDP) is pure Python: it has no FFI of its
 * own.  Each entry point below therefore names the reference call site whose sequence
 * of stock PyTorch ops it replaces; the Python mirror of the reference's comm-hook,
 * trainer and optimizer interfaces binds these symbols with ctypes.
 *
 * Conventions
 *  - Every function returns 0 on success and a negative JABAS_E* code on failure;
 *    jabas_last_error() then returns a message for the calling thread.
 *  - Every `float*` / `double*` data argument is a DEVICE pointer owned by the caller.
 *    Arrays of pointers (`const float* const*`) and all structs are HOST memory; they
 *    are consumed before the call returns.
 *  - `stream` is a cudaStream_t passed as void*.  Calls only enqueue work on it; they
 *    never synchronise the device and never block on the GPU.
 *  - Calls are thread-safe.  Calls that accumulate a statistic borrow a small
 *    reduction workspace that the context keeps per stream, so two such calls race
 *    only if the caller itself gives them the same `stat` accumulator on two streams.
 *  - There is no CPU fallback: without a CUDA device jabas_ctx_create() fails.
 */
#ifndef JABAS_B200_H
#define JABAS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define JABAS_API __attribute__((visibility("default")))
#else
#define JABAS_API
#endif

#define JABAS_B200_VERSION 1
#define JABAS_MAX_VSW      16   /* virtual stream workers (model replicas) per GPU */
#define JABAS_MAX_GROUPS   16   /* optimizer param groups per launch               */

#define JABAS_OK         0
#define JABAS_EINVAL    -1      /* bad argument (null, size, K, group index ...)   */
#define JABAS_ECUDA     -2      /* a CUDA runtime call failed                      */
#define JABAS_ENOMEM    -3      /* host or device allocation failed                */

typedef struct jabas_ctx    jabas_ctx_t;
typedef struct jabas_layout jabas_layout_t;
typedef struct jabas_dynhp  jabas_dynhp_t;

/* One run of consecutive elements of a flat parameter buffer that belongs to one
 * optimizer param group: the flat form of the group lists the reference builds at
 * examples/resnet50/main.py:340-349 and examples/vit/main.py:405-423. */
typedef struct {
    uint64_t begin;     /* first element (inclusive), in elements of the flat buffer */
    uint64_t end;       /* last element (exclusive)                                  */
    uint32_t group;     /* index into the `groups` array of the update call          */
    uint32_t reserved;
} jabas_seg_t;

/* Per-launch hyper-parameters of one param group: `param_groups[i]['lr']` is mutated
 * every iteration by the reference (jabas/train/trainer.py:693-700). */
typedef struct {
    double  lr;
    double  weight_decay;
    int64_t step;       /* Adam/AdamW: step count AFTER this update's increment      */
    int64_t reserved;
} jabas_group_t;

typedef struct {
    double momentum;
    double dampening;
    int    nesterov;
    int    first_step;  /* 1: momentum buffer is created from the gradient (m = d)   */
    const float* grad_scale;  /* DEVICE scalar, nullable: when *grad_scale < 1 the gradient is
                                 multiplied by it before the update (jabas_clip_coef)       */
    const jabas_dynhp_t* dynamic; /* nullable: the kernel reads lr / weight decay / flags from
                                 this device-resident block (see jabas_dynhp_create)        */
    int    remote_sources;    /* 1: some gradient pointer of the call is another GPU's memory (peer
                                 mapping): the kernel then loads per thread, never by bulk copy  */
    int    reserved;
} jabas_sgd_hp_t;

typedef struct {
    double beta1;
    double beta2;
    double eps;
    int    decoupled;   /* 1: AdamW (p *= 1 - lr*wd); 0: Adam (g += wd*p)            */
    int    reserved;
    const float* grad_scale;  /* as in jabas_sgd_hp_t */
    const jabas_dynhp_t* dynamic; /* as in jabas_sgd_hp_t */
    int    remote_sources;    /* as in jabas_sgd_hp_t */
    int    reserved2;
} jabas_adam_hp_t;

JABAS_API int         jabas_version(void);
JABAS_API const char* jabas_last_error(void);

/* Context: device id, SM count, per-stream reduction workspaces. */
JABAS_API int jabas_ctx_create(int device, jabas_ctx_t** ctx);
JABAS_API int jabas_ctx_destroy(jabas_ctx_t* ctx);

/* How the update kernels (jabas_sgd_momentum_f32, jabas_adam_f32 and their jabas_vsw_* forms)
 * bring a tile of their input streams on chip.  No reference counterpart: the reference's
 * updates are per-tensor PyTorch ops (examples/resnet50/main.py:351-359).
 *  - JABAS_STAGING_REGISTER (default): per-thread 128-bit loads straight into registers;
 *  - JABAS_STAGING_BULK: TMA bulk copies (cp.async.bulk) of 4 KB per stream into a multi-stage
 *    shared-memory ring, completion on mbarriers.  Results are bit-identical (the statistic to
 *    fp64 summation order).  Launches with hp->remote_sources set keep the register
 *    form.  Every wait on a copy is bounded by wall time (the GPU's global timer, 50 ms by
 *    default); a wait that runs out ends the CTA's loop early, at the same tile for all of its
 *    threads, and is counted (the launch's outputs are then incomplete).
 * jabas_ctx_set_staging allocates the 4-byte device counter the first time BULK is chosen.
 * jabas_ctx_staging_timeouts synchronises the device and reads the counter (0 = every launch
 * so far completed all of its copies). */
#define JABAS_STAGING_REGISTER 0
#define JABAS_STAGING_BULK     1
JABAS_API int jabas_ctx_set_staging(jabas_ctx_t* ctx, int mode);
JABAS_API int jabas_ctx_staging_timeouts(jabas_ctx_t* ctx, uint32_t* count);

/* Wall-time limits of the two kinds of device-side wait in this library, in milliseconds:
 * a CTA's wait for a bulk copy into its shared-memory ring (default 50), and a CTA's wait for
 * another GPU's progress inside the pipelined exchange (jabas_exchange_*; default 5000, which
 * has to absorb the skew between ranks).  A wait that runs out never traps: the kernel records
 * it and returns.  No reference counterpart. */
JABAS_API int jabas_ctx_set_wait_limits(jabas_ctx_t* ctx, double staging_ms, double peer_ms);

/* Test seam (host-side fault injection): when on, every stage barrier of the bulk-staged update
 * kernels expects 16 bytes more than are copied, so each CTA's first wait runs out after the
 * staging limit while every copy that was issued still completes.  Used to exercise the
 * time-out path without faulting the GPU; never set in production. */
JABAS_API int jabas_ctx_inject_staging_stall(jabas_ctx_t* ctx, int on);

/* Uploads a segment table covering [0, total) of a flat parameter buffer.  Segments
 * must be sorted, non-empty and contiguous (seg[i].end == seg[i+1].begin).
 * Synchronous (one small cudaMemcpy); call at set-up, not per iteration. */
JABAS_API int jabas_layout_create(jabas_ctx_t* ctx, const jabas_seg_t* segs, int nseg, uint64_t total,
                        jabas_layout_t** layout);
JABAS_API int jabas_layout_destroy(jabas_layout_t* layout);

/* Device-resident hyper-parameters, for update launches that are captured in a CUDA graph.
 * A graph bakes kernel arguments in, but the reference changes `lr` every iteration
 * (jabas/train/trainer.py:693-700) and Adam's step count grows.  An update call whose
 * hp->dynamic is set makes the kernel read those values from this block instead of from
 * its arguments.  Before every replay, OUTSIDE the graph, call jabas_dynhp_push_*: it
 * converts the hyper-parameters exactly as the update call would and enqueues a
 * 288-byte host-to-device copy on `stream` (from a ring of 8 pinned slots; it waits on the
 * host only if the copy issued 8 pushes ago has not completed).  create allocates. */
JABAS_API int jabas_dynhp_create(jabas_ctx_t* ctx, jabas_dynhp_t** out);
JABAS_API int jabas_dynhp_destroy(jabas_dynhp_t* h);
JABAS_API int jabas_dynhp_push_sgd(jabas_dynhp_t* h, const jabas_group_t* groups, int ngroups,
                         const jabas_sgd_hp_t* hp, void* stream);
JABAS_API int jabas_dynhp_push_adam(jabas_dynhp_t* h, const jabas_group_t* groups, int ngroups,
                          const jabas_adam_hp_t* hp, void* stream);

/* Local aggregation of the K VSW gradient buckets of one GPU.
 *   sum      = g[0] + g[1] + ... + g[K-1]       (fp32, ascending k: order is fixed)
 *   out      = sum / divisor                    (IEEE division; out may alias g[0])
 *   half_out = sum                              (nullable)
 *   stat3   += (<E,O>, |E|^2, |O|^2), E/O = sum of the even-/odd-index VSWs divided by
 *              half_divisor (nullable; the single-GPU form of the two-half statistic)
 * Replaces: the IIDP reducer's local aggregation behind the hook layout of
 * jabas/train/trainer.py:461-468, the `div_(T)` of iidp_allreduce_hook, and the
 * `detach().clone()` of jabas/ddp_comm_hooks/similarity_allreduce.py:28. */
JABAS_API int jabas_vsw_aggregate_f32(jabas_ctx_t* ctx, const float* const* grads, int K, float* out,
                            float* half_out, uint64_t n, float divisor, float half_divisor,
                            double* stat3, void* stream);

/* x /= divisor in place.  Replaces `div_(T/2)` at
 * jabas/ddp_comm_hooks/similarity_allreduce.py:32. */
JABAS_API int jabas_div_f32(jabas_ctx_t* ctx, float* x, uint64_t n, float divisor, void* stream);

/* Fused SGD(-momentum) update of n elements starting at element `base` of the flat
 * buffer that `layout` describes (layout == NULL: every element is in group 0), with
 * write-back of the new weights to all K replicas and, optionally, the two-half
 * statistic in the same pass:
 *   e = half[i] / half_divisor, o = 2*g[i] - e, stat3 += (<e,o>, |e|^2, |o|^2).
 * w[0] is the main replica (read and written); w[1..K-1] are written only.
 * m may be NULL iff hp->momentum == 0.  half and stat3 are both NULL or both set.
 * Replaces: torch.optim.SGD.step / ShardSGD.step(gradients)
 * (examples/resnet50/main.py:351-359), the weight copy main -> VSWs
 * (jabas/train/trainer.py:530-534) and, for the statistic, the cat / all_gather /
 * cosine_similarity of jabas/train/trainer.py:470-483. */
JABAS_API int jabas_sgd_momentum_f32(jabas_ctx_t* ctx, const float* g, float* const* w, int K, float* m,
                           uint64_t n, uint64_t base, const jabas_layout_t* layout,
                           const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* hp,
                           const float* half, float half_divisor, double* stat3, void* stream);

/* Fused Adam / AdamW update; same contract as jabas_sgd_momentum_f32.
 * Replaces: torch.optim.AdamW / ShardAdamW (examples/vit/main.py:433-437),
 * torch.optim.Adam (examples/gnmt/train.py:786-792) and the body of
 * ShardGNMTAdam.step (examples/gnmt/seq2seq/train/shard_optimizer.py:30-90). */
JABAS_API int jabas_adam_f32(jabas_ctx_t* ctx, const float* g, float* const* w, int K, float* m, float* v,
                   uint64_t n, uint64_t base, const jabas_layout_t* layout,
                   const jabas_group_t* groups, int ngroups, const jabas_adam_hp_t* hp,
                   const float* half, float half_divisor, double* stat3, void* stream);

/* Single-GPU form of the whole path in ONE pass: the Kg VSW gradients are summed in
 * registers (ascending k), divided by `divisor` (T) and fed straight to the optimizer
 * update, so the averaged gradient never makes a round trip through HBM: 4(Kg + K + 3)
 * bytes per element for SGD-momentum instead of 4(Kg + 1) + 4(K + 4).  Kg <= 8.
 *   grad_out  nullable: also store the averaged gradient (what jabas_vsw_aggregate_f32 writes)
 *   stat3     nullable: += the VSW-parity statistic (even-/odd-index VSW sums / half_divisor)
 * Results are bit-identical to jabas_vsw_aggregate_f32 followed by jabas_sgd_momentum_f32.
 * Only valid when no collective sits between aggregation and update (one GPU).
 * Replaces, in one launch: IIDP local aggregation + div_(T) + optimizer step
 * (examples/resnet50/main.py:351-359) + weight copy (jabas/train/trainer.py:530-534)
 * + cosine sums (jabas/train/trainer.py:470-483). */
JABAS_API int jabas_vsw_sgd_momentum_f32(jabas_ctx_t* ctx, const float* const* grads, int Kg, float divisor,
                               float* grad_out, float* const* w, int K, float* m, uint64_t n,
                               uint64_t base, const jabas_layout_t* layout, const jabas_group_t* groups,
                               int ngroups, const jabas_sgd_hp_t* hp, float half_divisor, double* stat3,
                               void* stream);

/* Adam / AdamW counterpart of jabas_vsw_sgd_momentum_f32 (examples/vit/main.py:433-437,
 * examples/gnmt/seq2seq/train/shard_optimizer.py:30-90). */
JABAS_API int jabas_vsw_adam_f32(jabas_ctx_t* ctx, const float* const* grads, int Kg, float divisor,
                       float* grad_out, float* const* w, int K, float* m, float* v, uint64_t n,
                       uint64_t base, const jabas_layout_t* layout, const jabas_group_t* groups,
                       int ngroups, const jabas_adam_hp_t* hp, float half_divisor, double* stat3,
                       void* stream);

/* stat3 += (<a,b>, |a|^2, |b|^2).  Replaces the three reductions inside
 * F.cosine_similarity at jabas/train/trainer.py:478. */
JABAS_API int jabas_dot_norms_f32(jabas_ctx_t* ctx, const float* a, const float* b, uint64_t n,
                        double* stat3, void* stream);

/* ---- The cross-GPU gradient path as ONE pipelined kernel per GPU --------------------------------
 *
 * Replaces, for one element range of the flat buffers, the whole per-bucket chain of the
 * reference: IIDP's local aggregation of the K VSW buckets, the sub-group and world allreduces
 * fired per bucket by the comm hook (jabas/ddp_comm_hooks/similarity_allreduce.py:20-45,
 * registered at jabas/train/trainer.py:327-337), the optimizer step, the weight copy to the VSW
 * replicas (jabas/train/trainer.py:530-534) and the sums of the cosine (:470-483).
 *
 * The range is cut into pieces of piece_elems elements, dealt to the ranks in turn (piece P is
 * reduced by rank P mod nranks).  One persistent kernel per GPU draws work items (aggregate /
 * reduce / update of one piece) from an ordered queue in which the reduce items of a window of
 * pieces stand one step behind its aggregate items and one step ahead of its update items, so
 * that NVLink-bound and HBM-bound work run together.  Ranks synchronise through per-piece epoch
 * flags stored into each other's flag blocks with plain peer stores; every wait is
 * bounded by the context's peer wait limit (jabas_ctx_set_wait_limits) and a wait that runs out is
 * reported through jabas_exchange_status, never by a trap.  Summation order is fixed: VSWs
 * ascending, then ranks ascending with each rank's sum divided by `divisor` first; E / O of the
 * statistic are the sums over even / odd ranks divided by `half_divisor`.  All ranks end with
 * bit-identical weights.
 *
 * Set-up: every rank owns three buffers that all ranks can address (peer mappings; the caller
 * allocates and exchanges them, e.g. with torch symmetric memory): `px` and `pg`, as long as the
 * flat buffers (fp32), and a flag block of jabas_exchange_flag_words(max_slots) uint32 that must be
 * zero before the first launch on ANY rank.  `max_slots` bounds slot_base + pieces of a launch;
 * launches of one iteration that cover different ranges (one per DDP bucket) use disjoint slots.
 * Every rank must issue the same sequence of launches.  Launches of one exchange must not overlap
 * on the GPU (keep them on one stream). */
#define JABAS_EXCHANGE_PIECE 8192u       /* default elements of one work item, per stream */
typedef struct jabas_exchange jabas_exchange_t;
typedef struct {
    int nranks;                     /* 2..8 */
    int rank;
    const float* const* px;         /* nranks device pointers, rank order (valid on this GPU) */
    const float* const* pg;
    uint32_t* const* flags;
    uint32_t max_slots;
    uint32_t window_pieces;         /* pieces per pipeline step; 0: sized from the launch grid */
    uint32_t piece_elems;           /* 0: JABAS_EXCHANGE_PIECE; else a multiple of 1024 */
    uint32_t update_lag;            /* pipeline steps between a piece's reduce item and its update items:
                                     * 1 or 2; 0: default.  Same value on every rank. */
} jabas_exchange_desc_t;

/* Per-rank buffers of a launch.  grads: Kg VSW gradient buffers; w: K weight replicas (w[0] is the
 * main replica); m, v: optimizer state; all indexed like the flat buffers (element `base` of the
 * launch is element `base` of each).  stat3 (nullable, device): += this rank's share of
 * (<E,O>, |E|^2, |O|^2). */
typedef struct {
    const float* const* grads;
    int Kg;
    int K;
    float* const* w;
    float* m;
    float* v;
    double* stat3;
} jabas_exchange_bufs_t;

JABAS_API size_t jabas_exchange_flag_words(uint32_t max_slots);
JABAS_API int jabas_exchange_create(jabas_ctx_t* ctx, const jabas_exchange_desc_t* desc, jabas_exchange_t** out);
JABAS_API int jabas_exchange_destroy(jabas_exchange_t* ex);
/* Synchronises the device and clears the exchange's local counters, launch counter and status (to
 * be followed by zeroing the flag blocks on every rank and a barrier: recovery after a time-out). */
JABAS_API int jabas_exchange_reset(jabas_exchange_t* ex);
/* Synchronous read of the status word (0 = no wait ever ran out; otherwise bit 31 set, bits 24..27
 * the phase that gave up: 2 reduce, 3 update, 4 statistic, bits 0..23 the piece slot) and, optionally,
 * of the number of completed launches. */
JABAS_API int jabas_exchange_status(jabas_exchange_t* ex, uint32_t* status, uint32_t* launches);

/* Kernel variant of the following launches: 2 resident CTAs per SM with a 96 KB ring each, 3 with a
 * 64 KB ring and 64 registers per thread, or 0 (default): 3 on two ranks with at most five streams per
 * stage, else 2 (measured choices, see exchange.cu). */
JABAS_API int jabas_exchange_set_ctas_per_sm(jabas_exchange_t* ex, int ctas);

/* Largest grid of the following launches (0, the default: every CTA the GPU can hold).  A launch
 * that shares the GPU with other work — the per-bucket launches fired during backward — should
 * leave shared memory and warp slots to it: CTAs of the exchange that wait for another rank hold
 * 96 KB of shared memory each while they wait.  One CTA per SM is a good limit there. */
JABAS_API int jabas_exchange_set_grid_limit(jabas_exchange_t* ex, uint32_t max_ctas);

/* Tracing (off by default; device_buf NULL turns it off).  Launches made while a buffer is set write
 * six uint64 per drawn ticket t < tickets at device_buf[6t]: (phase << 56 | CTA << 32 | piece), the
 * GPU's global-timer nanoseconds when the producer drew the ticket, when the item's flags had been
 * seen, when its last tile had been issued, when the consumers had stored its last tile, and one
 * spare word.  Tickets that hold no work stay untouched.  For timelines of the pipeline. */
JABAS_API int jabas_exchange_set_trace(jabas_exchange_t* ex, uint64_t* device_buf, uint64_t tickets);

/* One launch over elements [base, base + n) (both multiples of 4).  Exactly one of sgd / adam is
 * non-NULL; groups / layout as in jabas_sgd_momentum_f32.  nlocal == 1: exs[0] / bufs[0] are this
 * GPU's rank (the production form, one process per GPU).  nlocal == nranks: all ranks live on
 * this one GPU (exs[r] has rank r) and run as ONE launch sized so that every CTA is resident — the
 * form single-GPU tests of the protocol use; it synchronises the stream once. */
JABAS_API int jabas_exchange_step_f32(jabas_exchange_t* const* exs, const jabas_exchange_bufs_t* bufs, int nlocal,
                                      uint64_t n, uint64_t base, uint32_t slot_base, float divisor,
                                      float half_divisor, const jabas_layout_t* layout,
                                      const jabas_group_t* groups, int ngroups, const jabas_sgd_hp_t* sgd,
                                      const jabas_adam_hp_t* adam, void* stream);

/* After the launches of an iteration: every rank publishes its three sums to all ranks, waits
 * (bounded) for the others', adds them in rank order — stat3 then holds the sums over all ranks,
 * identical everywhere — and writes cos_out[0] = stat3[0] / sqrt(max(stat3[1]*stat3[2], eps^2)).
 * Replaces the all_gather / cosine_similarity / broadcast of jabas/train/trainer.py:470-483. */
JABAS_API int jabas_exchange_cosine(jabas_exchange_t* const* exs, double* const* stat3, float* const* cos_out,
                                    int nlocal, double eps, void* stream);

/* stat3[0..2] += sum of x[i]^2 (fp64).  First half of gradient-norm clipping:
 * clip_grad_norm_for_overlap at examples/gnmt/seq2seq/train/shard_optimizer.py:75-76 and
 * clip_grad_norm_ at examples/gnmt/seq2seq/train/trainer.py:157-161. */
JABAS_API int jabas_sumsq_f32(jabas_ctx_t* ctx, const float* x, uint64_t n, double* stat3, void* stream);

/* coef_out[0] = max_norm / (sqrt(sumsq[0]) + 1e-6) in fp32, coef_out[1] = the norm: the
 * clip coefficient of torch.nn.utils.clip_grad_norm_ (PyTorch v1.8.1).  Pass coef_out as
 * `grad_scale` of the update: the gradient is scaled only when the coefficient is < 1. */
JABAS_API int jabas_clip_coef(jabas_ctx_t* ctx, const double* sumsq, double max_norm, float* coef_out,
                    void* stream);

/* cos_out[0] = stat3[0] / sqrt(max(stat3[1]*stat3[2], eps^2)), evaluated in fp64.
 * Replaces the final division of F.cosine_similarity (jabas/train/trainer.py:478). */
JABAS_API int jabas_cosine_finalize(jabas_ctx_t* ctx, const double* stat3, double eps, float* cos_out,
                          void* stream);

/* dst[k][i] = src[i] for k < ndst (entries equal to src are skipped): one read of the
 * main replica, ndst writes.  Replaces the per-parameter copy loop of
 * jabas/train/trainer.py:530-534 (IIDP's `copy_time` stage). */
JABAS_API int jabas_replicate_f32(jabas_ctx_t* ctx, const float* src, float* const* dst, int ndst,
                        uint64_t n, void* stream);

/* No counterpart in the reference.  Same reduction as jabas_dot_norms_f32
 * (stat3 += (<a,b>, |a|^2, |b|^2)) for callers that cannot allocate device memory when
 * they need it: a process whose allocator already owns all of HBM, a section that must not
 * hit a synchronising cudaMalloc, a plugin without a context to keep a workspace in.
 * It takes no context and calls no cudaMalloc / cudaFree: the per-CTA partial sums live in
 * a static device array inside the library (about 48 KiB per GPU, held until exit).
 *  - n may not exceed JABAS_STATIC_MAX_ELEMS; larger inputs are refused with JABAS_EINVAL.
 *  - The first call on each device looks up the array's device address (a host-side query,
 *    made with that device current); make that first call before any stream capture begins.
 *  - All calls share the one array: two calls that overlap on the GPU (different streams,
 *    or different threads on different streams) race.  Keep them on one stream or order
 *    them with events. */
#define JABAS_STATIC_MAX_ELEMS (1ull << 31)
JABAS_API int jabas_dot_norms_static_f32(const float* a, const float* b, uint64_t n, double* stat3,
                                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JABAS_B200_H */
