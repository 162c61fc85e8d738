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
// The flat range is cut into pieces of `piece` elements, dealt to the ranks in turn (piece P is
// reduced by rank P mod n).  A piece of one phase is one work item.  Items stand in a queue
// ordered by pipeline step s = 0, 1, ...: with windows of W pieces, step s holds the aggregate
// items of window s, this rank's reduce items of window s-1 and the update items of window s-3
// (s-2 with update_lag 1), interleaved (one reduce item, then aggregate and update items in
// turn), so that at any moment
// the resident CTAs work on NVLink-bound and HBM-bound items together and the two resources
// overlap (the aggregate items run one window further ahead than this sketch says, see
// producer_loop).  CTAs draw items with an atomic ticket, in queue order.
//
// Dependencies are per-piece flags, not collectives: an aggregate item stores the launch's epoch
// into the flag block of the piece's owner; the owner's reduce item waits for the n flags of its
// piece and then stores the epoch into every rank's flag block; an update item waits for that
// flag.  An item only ever waits for items of earlier pipeline steps, and tickets are drawn
// in order, so every item a wait depends on is already held by a running CTA on its GPU: no
// deadlock, whatever the number of resident CTAs.  A reduce item's inputs were drawn two steps
// earlier, an update item's reduce item two steps earlier as well (measured on 4 GPUs: a reduce
// item takes about 40 us from its draw to the moment its flag is visible on the other GPUs — wait,
// issue, drain, 20-30 us of system-scope release under full HBM load —, more than one step of a
// ResNet-50-sized launch; with one step of distance the update items waited 6 us on average and
// 25-33 us at the 95th percentile, with two 3 us and 17-20 us).  Every wait is bounded by wall
// time; a wait that
// runs out records (phase, slot) in a status word, all CTAs of the launch drain, and the host
// reads the status — the kernel never traps and never spins for ever.
//
// Summation order is fixed (VSWs ascending, then ranks ascending, each term divided by T first:
// the reference's div_(T) before the SUM allreduce), so every rank computes bit-identical
// gradients and weights.  Tiles come on chip by bulk copies without multicast (cp.async.bulk,
// from local or peer memory), flags go out as plain peer stores: no multicast anywhere.
#include "common.cuh"

#include <algorithm>
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
    double* piece_stat;                 // local: [max_slots][3], written for the pieces this rank reduces
    double* stat;                       // nullable: += this launch's (<E,O>, |E|^2, |O|^2) over this rank's shards
    const SegDev* segs;
    unsigned long long base, n;         // element range of the launch
    unsigned long long wait_ns;
    unsigned long long npieces;         // pieces of the launch
    unsigned int piece, window, nsteps, slot_base, max_slots;   // piece: elements of an item; window: pieces per step
    unsigned int total_tickets;         // length of the queue
    unsigned int upd_lag;               // steps an update item stands behind its reduce item (1 or 2)
    int nseg, K, Kw, nranks, rank;
    int opt;                            // OPT_SGD / OPT_ADAM
    int ring_stages, ring_slots;        // shared-memory ring: stages, and 4 KB stream slots per stage
    float divisor, half_divisor;
    const UpdHp* dyn;
    unsigned long long* trace;          // nullable: 6 words per ticket (see jabas_exchange_set_trace)
    unsigned long long trace_cap;       // tickets the trace buffer holds
    UpdHp hp;
};

}  // namespace jb_types

namespace {

// A CTA is 8 consumer warps, one producer warp and one publisher warp (one active lane each).  The producer (one lane) draws tickets, waits
// for the item's flags and brings the item on chip tile by tile with bulk copies (TMA, no
// multicast; the source may be another GPU's memory) into a ring of shared-memory stages; it runs
// up to a ring ahead of the consumers, ACROSS items, so neither the flag polls nor the first-byte
// latency of an item (several microseconds over NVLink) ever leave the memory pipes idle.  The
// consumers read a stage into registers, free it, do the arithmetic and the stores, and after an
// item's last tile hand the item to the publisher — independently of the producer, which may by
// then be blocked on a flag of a later item (so that wait can never stall what it waits for).
// The publisher does the system-scope release and the flag stores: the release has to wait until
// the item's stores have drained (measured: 6-11 us under full HBM load), which would otherwise
// stall a consumer warp, and with it the ring, once per item.
constexpr int kConsumers = kThreads;                     // 256
constexpr int kExThreads = kThreads + 64;                // + the producer warp + the publisher warp
constexpr int kMailSlots = 8;
constexpr int kTileVecs = kThreads;                      // one 4-vector per consumer thread and stream
constexpr unsigned kTileBytes = kTileVecs * 16;          // 4 KB per stream and stage
constexpr unsigned kTileElems = kTileVecs * 4;
constexpr int kExMaxStages = 8;
constexpr int kExMaxSlots = 8;                           // streams of a stage: K gradients, n sums, or g/p/m/v
constexpr int kRingBudgetBytes = 96 * 1024;              // dynamic shared memory per CTA (two CTAs per SM)

enum { CTL_QUEUE = 0, CTL_DONE = 32, CTL_LAUNCHES = 64, CTL_STATUS = 96, CTL_STAT_EPOCH = 128, CTL_WORDS = 160 };
enum { PH_STOP = 0, PH_AGG = 1, PH_RED = 2, PH_UPD = 3, PH_STAT = 4, PH_RING = 5 };

// flag block of a rank: [max_slots][8] aggregate flags (one per source rank), [max_slots] reduce
// flags, then (on a 32-byte boundary) 8 statistic slots of 8 words
__host__ __device__ inline size_t stat_base(unsigned max_slots) { return ((size_t)max_slots * (kExMaxRanks + 1) + 7) / 8 * 8; }
__host__ __device__ inline size_t flag_words(unsigned max_slots) { return stat_base(max_slots) + 8 * kExMaxRanks; }
__device__ __forceinline__ unsigned agg_flag_idx(unsigned slot, int src) { return slot * kExMaxRanks + src; }
__device__ __forceinline__ unsigned red_flag_idx(unsigned max_slots, unsigned slot) { return max_slots * kExMaxRanks + slot; }
__device__ __forceinline__ unsigned stat_idx(unsigned max_slots, int src) { return (unsigned)stat_base(max_slots) + src * 8; }

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile(const unsigned* p)
{
    return *reinterpret_cast<const volatile unsigned*>(p);
}
// barrier among the 256 consumer threads only (the producer warp never joins it)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

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

// All n flags of a piece.  Every poll is an acquire LOAD (measured: 0.3 us each under full load);
// a relaxed poll followed by one system-scope acquire FENCE cost 11 us per item, because the
// fence waits for the SM's outstanding stores to drain although the polling lane has none.
__device__ __forceinline__ bool wait_epoch_n(const unsigned* f, int n, unsigned epoch, unsigned long long limit_ns,
                                             const unsigned* status)
{
    unsigned long long t0 = 0;
    int r = 0;                                   // flags 0..r-1 have been seen
    for (unsigned long long polls = 0;; ++polls) {
        while (r < n && (int)(ld_acquire_sys(f + r) - epoch) >= 0) ++r;
        if (r == n) return true;
        if (polls == 0) t0 = gtime_ns();
        __nanosleep(40);
        if ((polls & 7) == 7) {
            if (gtime_ns() - t0 > limit_ns || polls > limit_ns / 64 + 4096) return false;
            if (ld_volatile(status) != 0u) return false;
        }
    }
}

// A wait ran out: record where (first one wins) and set the top bit of the ticket counter, so
// that every later draw lies past the end of the queue.
constexpr unsigned kQueueAbort = 0x80000000u;
__device__ __forceinline__ void record_timeout(const ExArgs& a, int phase, unsigned slot)
{
    atomicCAS(a.ctrl + CTL_STATUS, 0u, 0x80000000u | ((unsigned)phase << 24) | (slot & 0xffffffu));
    atomicOr(a.ctrl + CTL_QUEUE, kQueueAbort);
}

struct TileDesc {
    unsigned long long lo;      // first element of the tile in the flat buffers
    unsigned nvec;              // 4-vectors in the tile (<= 256)
    int phase;                  // PH_STOP ends the consumers' loop
    int owner;
    unsigned slot;
    int last;                   // last tile of its item
    unsigned ticket;
};

struct Mail {
    unsigned slot, ticket;
    int owner, phase;           // PH_AGG / PH_RED: publish that piece; PH_STOP: leave
};

struct ExShared {
    ExArgs a;
    UpdHp H;
    Mail mail[kMailSlots];
    unsigned mail_head;         // written by consumer thread 0 (release), read by the publisher (acquire)
    volatile unsigned mail_tail;
    unsigned long long full[kExMaxStages];
    unsigned long long empty[kExMaxStages];
    TileDesc desc[kExMaxStages];
    double red[3][kWarps];
    int is_last;
    volatile int producer_done;
};

// ---- producer: one lane ---------------------------------------------------------------------
__device__ __noinline__ void producer_loop(ExShared& S, unsigned char* ring, unsigned epoch)
{
    const ExArgs& a = S.a;
    const int n = a.nranks;
    const unsigned group_items = 2u * (unsigned)n + 1u;
    // The queue opens with the aggregate items of window 0 alone; after that, step s holds the
    // aggregate items of window s+1, the reduce items of window s-1 and the update items of window
    // s-ulag.  Aggregation has no dependencies, so it runs a window further ahead than the pipeline
    // needs: a reduce item's flags take about 30 us from the draw of the matching aggregate item
    // (issue, drain of the stores behind the system-scope release, NVLink), and without the lead
    // the reduce items of the first window would be drawn before that.
    // Steps hold only the phases that have a window to work on (the first and the last two steps
    // lack some), so no ticket is drawn for nothing: a ticket costs an atomic's round trip.
    const unsigned prologue = a.npieces < a.window ? (unsigned)a.npieces : a.window;
    const unsigned groups = a.window / (unsigned)n;
    const unsigned nsteps = a.nsteps;
    const unsigned ulag = 1u + a.upd_lag;          // update items of window w stand in step w + ulag
    auto has_r = [&](unsigned st) { return st >= 1u && st <= nsteps; };
    auto has_a = [&](unsigned st) { return st + 1u < nsteps; };
    auto has_u = [&](unsigned st) { return st >= ulag && st < nsteps + ulag; };
    auto group_len = [&](unsigned st) {
        return (has_r(st) ? 1u : 0u) + (has_a(st) ? (unsigned)n : 0u) + (has_u(st) ? (unsigned)n : 0u);
    };
    const unsigned total = a.total_tickets;
    const unsigned long long end = a.base + a.n;
    const unsigned* status = a.ctrl + CTL_STATUS;
    const unsigned* flags_local = a.flags[a.rank];
    const bool load_m = a.opt == OPT_ADAM || ((S.H.flags & F_MOMENTUM) && !(S.H.flags & F_FIRST));
    const size_t stage_bytes = (size_t)a.ring_slots * kTileBytes;
    int stage = 0;
    unsigned parity = 0;            // phase of the empty barriers this lane waits for next
    bool ok = true;
    unsigned t = atomicAdd(a.ctrl + CTL_QUEUE, 1u);
    while (ok && t < total) {
        const unsigned nxt = atomicAdd(a.ctrl + CTL_QUEUE, 1u);      // resolves while this item is issued
        int phase;
        long long win;
        unsigned idx;
        if (t < prologue) { phase = PH_AGG; win = 0; idx = t; }
        else {
            unsigned tq = t - prologue, step = 0;
            bool found = false;
            for (; step < ulag; ++step) {                      // the first steps are short
                const unsigned len = groups * group_len(step);
                if (tq < len) { found = true; break; }
                tq -= len;
            }
            if (!found && nsteps >= ulag + 2u) {               // steps ulag .. nsteps-2 hold all three phases
                const unsigned len = groups * group_items, nfull = nsteps - 1u - ulag;
                if (tq < nfull * len) { step = ulag + tq / len; tq %= len; found = true; }
                else { tq -= nfull * len; step = nsteps - 1u; }
            }
            for (; !found && step < nsteps + ulag; ++step) {   // the last steps are short again
                const unsigned len = groups * group_len(step);
                if (tq < len) { found = true; break; }
                tq -= len;
            }
            const unsigned glen = group_len(step);
            const unsigned grp = tq / glen;
            unsigned i = tq % glen;
            if (has_r(step) && i == 0u) { phase = PH_RED; win = (long long)step - 1; idx = grp * (unsigned)n + (unsigned)a.rank; }
            else {
                if (has_r(step)) --i;
                if (has_a(step) && has_u(step)) {
                    idx = grp * (unsigned)n + (i >> 1);
                    if (i & 1u) { phase = PH_UPD; win = (long long)step - (long long)ulag; } else { phase = PH_AGG; win = (long long)step + 1; }
                } else {
                    idx = grp * (unsigned)n + i;
                    if (has_a(step)) { phase = PH_AGG; win = (long long)step + 1; } else { phase = PH_UPD; win = (long long)step - (long long)ulag; }
                }
            }
        }
        const unsigned long long P = (unsigned long long)(win < 0 ? 0 : win) * a.window + idx;
        if (win >= 0 && win < (long long)a.nsteps && P < a.npieces) {
            const unsigned slot = a.slot_base + (unsigned)P;
            const int owner = (int)(P % (unsigned)n);
            const unsigned long long lo = a.base + P * a.piece;
            unsigned long long hi = lo + a.piece;
            if (hi > end) hi = end;
            unsigned long long* tr = (a.trace && t < a.trace_cap) ? a.trace + 6ull * t : nullptr;
            if (tr) { tr[0] = ((unsigned long long)phase << 56) | ((unsigned long long)blockIdx.x << 32) | (unsigned)P; tr[1] = gtime_ns(); }
            if (phase == PH_RED) {
                ok = wait_epoch_n(flags_local + agg_flag_idx(slot, 0), n, epoch, a.wait_ns, status);
                if (!ok) record_timeout(a, PH_RED, slot);
            } else if (phase == PH_UPD) {
                ok = wait_epoch(flags_local + red_flag_idx(a.max_slots, slot), epoch, a.wait_ns, status);
                if (!ok) record_timeout(a, PH_UPD, slot);
            }
            if (tr) tr[2] = gtime_ns();
            for (unsigned long long e0 = lo; ok && e0 < hi; e0 += kTileElems) {
                if (!mbar_wait_bounded(&S.empty[stage], parity ^ 1u, 2 * a.wait_ns + 10000000ull)) {
                    record_timeout(a, PH_RING, slot);
                    ok = false;
                    break;
                }
                const unsigned long long left = hi - e0;
                const unsigned nvec = left >= kTileElems ? (unsigned)kTileVecs : (unsigned)(left >> 2);
                const unsigned bytes = nvec * 16u;
                TileDesc& d = S.desc[stage];
                d.lo = e0; d.nvec = nvec; d.phase = phase; d.owner = owner; d.slot = slot;
                d.last = e0 + kTileElems >= hi;
                d.ticket = t;
                unsigned char* sb = ring + (size_t)stage * stage_bytes;
                fence_proxy_async_smem();
                if (phase == PH_AGG) {
                    mbar_expect_tx(&S.full[stage], bytes * (unsigned)a.K);
                    for (int k = 0; k < a.K; ++k) bulk_load(sb + k * kTileBytes, a.gk[k] + e0, bytes, &S.full[stage]);
                } else if (phase == PH_RED) {
                    mbar_expect_tx(&S.full[stage], bytes * (unsigned)n);
                    for (int r = 0; r < n; ++r) bulk_load(sb + r * kTileBytes, a.px[r] + e0, bytes, &S.full[stage]);
                } else {
                    const unsigned ns = 2u + (load_m ? 1u : 0u) + (a.opt == OPT_ADAM ? 1u : 0u);
                    mbar_expect_tx(&S.full[stage], bytes * ns);
                    bulk_load(sb, a.pg[owner] + e0, bytes, &S.full[stage]);
                    bulk_load(sb + kTileBytes, a.w[0] + e0, bytes, &S.full[stage]);
                    if (load_m) bulk_load(sb + 2 * kTileBytes, a.m + e0, bytes, &S.full[stage]);
                    if (a.opt == OPT_ADAM) bulk_load(sb + 3 * kTileBytes, a.v + e0, bytes, &S.full[stage]);
                }
                if (++stage == a.ring_stages) { stage = 0; parity ^= 1u; }
            }
            if (tr) tr[3] = gtime_ns();
        }
        t = nxt;
    }
    // end of the queue (or a wait ran out): one last descriptor tells the consumers to leave
    if (mbar_wait_bounded(&S.empty[stage], parity ^ 1u, 2 * a.wait_ns + 10000000ull)) {
        S.desc[stage].phase = PH_STOP;
        mbar_arrive(&S.full[stage]);
    }
    S.producer_done = 1;
}

__device__ __forceinline__ unsigned ld_acquire_cta_shared(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_cta_shared(unsigned* p, unsigned v)
{
    asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

// consumer thread 0, after the consumers' barrier that follows an item's last stores
__device__ __forceinline__ void mail_push(ExShared& S, int phase, int owner, unsigned slot, unsigned ticket)
{
    const unsigned head = S.mail_head;
    while (head - S.mail_tail >= (unsigned)kMailSlots) __nanosleep(20);
    Mail& m = S.mail[head % kMailSlots];
    m.slot = slot; m.ticket = ticket; m.owner = owner; m.phase = phase;
    st_release_cta_shared(&S.mail_head, head + 1u);      // orders the entry (and, through the barrier, the item's stores)
}

// ---- publisher: one lane ----------------------------------------------------------------------
__device__ __noinline__ void publisher_loop(ExShared& S, unsigned epoch)
{
    const ExArgs& a = S.a;
    const int n = a.nranks;
    unsigned tail = 0;
    unsigned long long idle_since = 0;
    for (;;) {
        const unsigned head = ld_acquire_cta_shared(&S.mail_head);
        if (head == tail) {
            // nothing to publish: the consumers always end with a stop entry; the time limit only
            // guards against that never coming
            if (idle_since == 0) idle_since = gtime_ns();
            else if (gtime_ns() - idle_since > 8 * a.wait_ns + 100000000ull) return;
            __nanosleep(50);
            continue;
        }
        idle_since = 0;
        // Everything that is waiting goes out behind ONE system-scope fence: the fence has to wait
        // for the items' stores to drain, and entries pile up meanwhile.  The acquire above and the
        // consumers' barrier before each push put every store of these items before the fence.
        Mail batch[kMailSlots];
        int nb = 0;
        bool stop = false;
        while (tail != head && nb < kMailSlots) {
            batch[nb] = S.mail[tail % kMailSlots];
            ++tail;
            if (batch[nb].phase == PH_STOP) { stop = true; break; }
            ++nb;
        }
        S.mail_tail = tail;
        if (nb > 0) {
            fence_acq_rel_sys();
            for (int b = 0; b < nb; ++b) {
                const Mail& m = batch[b];
                if (m.phase == PH_AGG) {
                    st_relaxed_sys(a.flags[m.owner] + agg_flag_idx(m.slot, a.rank), epoch);
                } else {
                    for (int r = 0; r < n; ++r) st_relaxed_sys(a.flags[r] + red_flag_idx(a.max_slots, m.slot), epoch);
                }
            }
            if (a.trace) {
                const unsigned long long now = gtime_ns();
                for (int b = 0; b < nb; ++b)
                    if (batch[b].ticket < a.trace_cap) a.trace[6ull * batch[b].ticket + 5] = now;
            }
        }
        if (stop) return;
    }
}

// CTA-wide (consumers only) sum, valid in consumer thread 0
__device__ __forceinline__ Acc3 consumer_sum(Acc3 v, double (*sm)[kWarps])
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    consumer_sync();
    if (lane == 0) { sm[0][warp] = v.d; sm[1][warp] = v.a; sm[2][warp] = v.b; }
    consumer_sync();
    Acc3 r = {0.0, 0.0, 0.0};
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { r.d += sm[0][w]; r.a += sm[1][w]; r.b += sm[2][w]; }
    }
    return r;
}

// ---- consumers: 256 threads, one 4-vector per thread, stream and tile --------------------------
template <int OPT>
__device__ __forceinline__ void consumer_loop(ExShared& S, const unsigned char* ring, unsigned epoch)
{
    const ExArgs& a = S.a;
    const UpdHp& H = S.H;
    const int n = a.nranks;
    const bool use_m = OPT == OPT_ADAM || (H.flags & F_MOMENTUM);
    const bool load_m = OPT == OPT_ADAM || ((H.flags & F_MOMENTUM) && !(H.flags & F_FIRST));
    const bool stat = a.stat != nullptr;
    const size_t stage_bytes = (size_t)a.ring_slots * kTileBytes;
    const unsigned tid = threadIdx.x;
    int stage = 0;
    unsigned parity = 0;
    Acc3 acc = {0.0, 0.0, 0.0};
    for (;;) {
        if (!mbar_wait_bounded(&S.full[stage], parity, 4 * a.wait_ns + 20000000ull)) {
            if (tid == 0) record_timeout(a, PH_RING, 0);
            break;
        }
        const TileDesc d = S.desc[stage];
        if (d.phase == PH_STOP) break;
        const float4* sb = reinterpret_cast<const float4*>(ring + (size_t)stage * stage_bytes);
        const bool mine = tid < d.nvec;
        const unsigned long long off = d.lo + 4ull * tid;
        if (d.phase == PH_AGG) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mine) {
                s = sb[tid];
                for (int k = 1; k < a.K; ++k) s = add4(s, sb[k * kTileVecs + tid]);
            }
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&S.empty[stage]);       // the stage may be refilled
            if (mine) st4(a.px_local + off, s);
        } else if (d.phase == PH_RED) {
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f), e = g, o = g;
            if (mine) {
                e = sb[tid];
                g = div4(e, a.divisor);
                for (int r = 1; r < n; ++r) {
                    const float4 y = sb[r * kTileVecs + tid];
                    g = add4(g, div4(y, a.divisor));
                    if (r == 1) o = y; else if (r & 1) o = add4(o, y); else e = add4(e, y);
                }
            }
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&S.empty[stage]);
            if (mine) {
                st4(a.pg_local + off, g);
                if (stat) acc_vec(acc, div4(e, a.half_divisor), div4(o, a.half_divisor));
            }
        } else {
            float4 g, p, m, v;
            g = p = m = v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mine) {
                g = sb[tid];
                p = sb[kTileVecs + tid];
                if (load_m) m = sb[2 * kTileVecs + tid];
                if (OPT == OPT_ADAM) v = sb[3 * kTileVecs + tid];
            }
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&S.empty[stage]);
            // segment of the tile's first element, uniform over the CTA
            int seg0 = 0, gi0 = 0;
            bool uniform = true;
            if (a.segs) {
                const unsigned long long e1 = d.lo + 4ull * d.nvec;
                seg0 = seg_find(a.segs, a.nseg, d.lo);
                uniform = __ldg(&a.segs[seg0].end) >= e1;
                gi0 = (int)__ldg(&a.segs[seg0].group);
            }
            if (mine) {
                if (uniform) {
                    upd_math4<OPT>(H, H.grp[gi0], (H.wd_mask >> gi0) & 1u, g, p, m, v);
                } else {
                    int sgi = seg0;
                    auto one = [&](int c, float gx, float& px, float& mx, float& vx) {
                        while (__ldg(&a.segs[sgi].end) <= off + c) ++sgi;
                        const int gi = (int)__ldg(&a.segs[sgi].group);
                        upd_math<OPT>(H, H.grp[gi], (H.wd_mask >> gi) & 1u, gx, px, mx, vx);
                    };
                    one(0, g.x, p.x, m.x, v.x);
                    one(1, g.y, p.y, m.y, v.y);
                    one(2, g.z, p.z, m.z, v.z);
                    one(3, g.w, p.w, m.w, v.w);
                }
                for (int k = 0; k < a.Kw; ++k) st4(a.w[k] + off, p);
                if (use_m) st4(a.m + off, m);
                if (OPT == OPT_ADAM) st4(a.v + off, v);
            }
        }
        if (d.last && a.trace && tid == 64 && d.ticket < a.trace_cap) a.trace[6ull * d.ticket + 4] = gtime_ns();
        if (d.last && d.phase != PH_UPD) {
            // the item is complete once every consumer has issued its stores: one thread publishes
            // it, with release semantics that cover the stores the barrier made visible to it
            if (d.phase == PH_RED && stat) {
                const Acc3 r = consumer_sum(acc, S.red);
                if (tid == 0) {
                    double* ps = a.piece_stat + 3ull * d.slot;
                    ps[0] = r.d; ps[1] = r.a; ps[2] = r.b;
                }
                acc.d = acc.a = acc.b = 0.0;
            }
            consumer_sync();
            if (tid == 0) mail_push(S, d.phase, d.owner, d.slot, d.ticket);
        }
        if (++stage == a.ring_stages) { stage = 0; parity ^= 1u; }
    }
}

// One rank's share of a launch.  `ncta` CTAs of the grid (blockIdx.x) serve this rank.
template <int OPT>
__device__ __forceinline__ void exchange_body(ExShared& S, unsigned char* ring, unsigned ncta)
{
    const ExArgs& a = S.a;
    if (a.dyn) {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(a.dyn);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&S.H);
        for (unsigned int i = threadIdx.x; i < sizeof(UpdHp) / 4; i += blockDim.x) dst[i] = __ldg(src + i);
    } else {
        const unsigned int* src = reinterpret_cast<const unsigned int*>(&a.hp);
        unsigned int* dst = reinterpret_cast<unsigned int*>(&S.H);
        for (unsigned int i = threadIdx.x; i < sizeof(UpdHp) / 4; i += blockDim.x) dst[i] = src[i];
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kExMaxStages; ++s) {
            mbar_init(&S.full[s], 1);              // the producer's arrive (+ the copies' bytes)
            mbar_init(&S.empty[s], kWarps);        // one arrive per consumer warp
        }
        S.producer_done = 0;
        S.mail_head = 0;
        S.mail_tail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Every CTA reads the launch counter before its producer draws the first ticket; the counter
    // moves only when the last CTA of the launch leaves, i.e. after every CTA has read it.
    const unsigned epoch = ld_volatile(a.ctrl + CTL_LAUNCHES) + 1u;
    __syncthreads();                               // the only barrier all 320 threads share
    if (threadIdx.x >= kConsumers) {
        if (threadIdx.x == kConsumers) producer_loop(S, ring, epoch);
        else if (threadIdx.x == kConsumers + 32) publisher_loop(S, epoch);
        return;
    }
    consumer_loop<OPT>(S, ring, epoch);
    if (threadIdx.x == 0) mail_push(S, PH_STOP, 0, 0, 0);
    // Leaving.  Normally the stop descriptor was consumed and nothing is in flight.  After a wait
    // that ran out, give the producer (bounded) time to stop issuing before the CTA's shared
    // memory goes away.
    consumer_sync();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = gtime_ns();
        while (!S.producer_done && gtime_ns() - t0 < 6 * a.wait_ns + 50000000ull) __nanosleep(200);
        __threadfence();
        S.is_last = atomicAdd(a.ctrl + CTL_DONE, 1u) == ncta - 1u;
    }
    consumer_sync();
    if (!S.is_last) return;
    // the last CTA to leave adds this launch's piece sums in piece order, rewinds the queue and
    // advances the launch counter
    __threadfence();
    if (a.stat) {
        Acc3 s = {0.0, 0.0, 0.0};
        if (ld_volatile(a.ctrl + CTL_STATUS) == 0u) {
            for (unsigned long long q = (unsigned long long)a.rank + (unsigned long long)a.nranks * threadIdx.x;
                 q < a.npieces; q += (unsigned long long)a.nranks * kConsumers) {
                const double* ps = a.piece_stat + 3ull * (a.slot_base + q);
                s.d += __ldcg(ps + 0); s.a += __ldcg(ps + 1); s.b += __ldcg(ps + 2);
            }
        }
        s = consumer_sum(s, S.red);
        if (threadIdx.x == 0) { a.stat[0] += s.d; a.stat[1] += s.a; a.stat[2] += s.b; }
    }
    if (threadIdx.x == 0) {
        a.ctrl[CTL_QUEUE] = 0u;
        a.ctrl[CTL_DONE] = 0u;
        a.ctrl[CTL_LAUNCHES] = epoch;
    }
}

__device__ __forceinline__ void stage_args(ExArgs* dst, const ExArgs* src)
{
    const unsigned int* s = reinterpret_cast<const unsigned int*>(src);
    unsigned int* d = reinterpret_cast<unsigned int*>(dst);
    for (unsigned int i = threadIdx.x; i < sizeof(ExArgs) / 4; i += blockDim.x) d[i] = s[i];
    __syncthreads();
}

// MINB: resident CTAs per SM the kernel is compiled for (2: 96 KB ring, up to 128 registers;
// 3: 64 KB ring, 64 registers).
template <int OPT, int MINB>
__global__ void __launch_bounds__(kExThreads, MINB) exchange_kernel(const ExArgs arg)
{
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ ExShared S;
    stage_args(&S.a, &arg);
    exchange_body<OPT>(S, ring, gridDim.x);
}

// Several ranks' exchanges in ONE launch on ONE GPU (blockIdx.y = rank): kernels that wait on
// one another may not run as separate launches on a GPU, so single-GPU tests of the protocol
// use this form, with the grid sized so that every CTA is resident.
template <int OPT, int MINB>
__global__ void __launch_bounds__(kExThreads, MINB) exchange_emu_kernel(const ExArgs* ranks)
{
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ ExShared S;
    stage_args(&S.a, ranks + blockIdx.y);
    exchange_body<OPT>(S, ring, gridDim.x);
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
    unsigned long long* trace = nullptr;
    unsigned long long trace_cap = 0;
    unsigned grid_limit = 0;             // 0: every resident CTA of the GPU
    int ctas_per_sm = 0;                 // kernel variant: 2 (96 KB ring), 3 (64 KB ring), 0: by stream count
    jabas_ctx_t* ctx = nullptr;
    int nranks = 0, rank = 0;
    unsigned max_slots = 0, window = 0, piece = JABAS_EXCHANGE_PIECE;
    unsigned upd_lag = 2;                // steps between a piece's reduce item and its update items
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
    if (d->window_pieces > (1u << 20)) return fail(JABAS_EINVAL, "exchange: window_pieces out of range");
    if (d->piece_elems && (d->piece_elems % 1024u || d->piece_elems > (1u << 22)))
        return fail(JABAS_EINVAL, "exchange: piece_elems must be a multiple of 1024, at most 2^22 (0: default)");
    if (!d->px || !d->pg || !d->flags) return fail(JABAS_EINVAL, "exchange: null buffer table");
    if (d->update_lag > 2u) return fail(JABAS_EINVAL, "exchange: update_lag is 0 (default), 1 or 2");
    jabas_exchange_t* ex = new (std::nothrow) jabas_exchange_t();
    if (!ex) return fail(JABAS_ENOMEM, "out of host memory");
    ex->ctx = ctx; ex->nranks = d->nranks; ex->rank = d->rank; ex->max_slots = d->max_slots;
    ex->window = d->window_pieces;
    ex->upd_lag = d->update_lag ? d->update_lag : 2u;
    ex->piece = d->piece_elems ? d->piece_elems : JABAS_EXCHANGE_PIECE;
    for (int r = 0; r < d->nranks; ++r) {
        if (!d->px[r] || !d->pg[r] || !d->flags[r] || !aligned16(d->px[r]) || !aligned16(d->pg[r]) ||
            !aligned16(d->flags[r])) {
            delete ex;
            return fail(JABAS_EINVAL, "exchange: buffers must be non-null and 16-byte aligned");
        }
        ex->px[r] = d->px[r]; ex->pg[r] = d->pg[r]; ex->flags[r] = d->flags[r];
    }
    const size_t stat_off = ((size_t)CTL_WORDS * 4 + 255) / 256 * 256;
    ex->local_bytes = stat_off + sizeof(double) * 3 * (size_t)ex->max_slots;
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

int jabas_exchange_set_ctas_per_sm(jabas_exchange_t* ex, int ctas)
{
    if (!ex) return fail(JABAS_EINVAL, "exchange is null");
    if (ctas != 0 && ctas != 2 && ctas != 3) return fail(JABAS_EINVAL, "exchange: 2 or 3 CTAs per SM (0: automatic)");
    ex->ctas_per_sm = ctas;
    return JABAS_OK;
}

int jabas_exchange_set_grid_limit(jabas_exchange_t* ex, uint32_t max_ctas)
{
    if (!ex) return fail(JABAS_EINVAL, "exchange is null");
    ex->grid_limit = max_ctas;
    return JABAS_OK;
}

int jabas_exchange_set_trace(jabas_exchange_t* ex, uint64_t* device_buf, uint64_t tickets)
{
    if (!ex) return fail(JABAS_EINVAL, "exchange is null");
    ex->trace = reinterpret_cast<unsigned long long*>(device_buf);
    ex->trace_cap = device_buf ? tickets : 0;
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

static int fill_args(jabas_exchange_t* ex, unsigned grid_ctas, const jabas_exchange_bufs_t& b, ExArgs& a, uint64_t n, uint64_t base,
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
    a.trace = ex->trace; a.trace_cap = ex->trace_cap;
    a.piece_stat = reinterpret_cast<double*>(reinterpret_cast<char*>(ex->d_local) + ((size_t)CTL_WORDS * 4 + 255) / 256 * 256);
    a.base = base; a.n = n;
    a.wait_ns = (unsigned long long)(ctx->peer_wait_ms * 1e6);
    a.piece = ex->piece;
    a.npieces = (n + ex->piece - 1) / ex->piece;
    if ((unsigned long long)slot_base + a.npieces > ex->max_slots)
        return fail(JABAS_EINVAL, "exchange: the range needs more flag slots than the exchange was created with");
    // pieces per pipeline step: as asked, or so that a step holds about four items per CTA of the
    // grid — a consumer item then stands four rounds of tickets behind its producer item, which
    // has finished by then on every rank (measured: waits vanish from about three rounds on)
    unsigned long long window = ex->window;
    if (window == 0) window = (4ull * grid_ctas * ex->nranks) / (2ull * ex->nranks + 1);
    window = window / ex->nranks * ex->nranks;
    if (window < (unsigned long long)ex->nranks) window = ex->nranks;
    const unsigned long long nsteps = (a.npieces + window - 1) / window;
    const unsigned long long ulag = 1ull + ex->upd_lag;
    if (window + (nsteps + ulag) * (window / ex->nranks) * (2ull * ex->nranks + 1) >= 0x7ffffff0ull)
        return fail(JABAS_EINVAL, "exchange: too many work items for one launch");
    a.window = (unsigned)window; a.nsteps = (unsigned)nsteps; a.slot_base = slot_base; a.max_slots = ex->max_slots;
    {
        // length of the queue: the aggregate items of window 0, then per step only the phases that
        // have a window (see producer_loop)
        unsigned long long tickets = a.npieces < window ? a.npieces : window;
        const unsigned long long groups = window / ex->nranks;
        for (unsigned long long st = 0; st < nsteps + ulag; ++st) {
            const unsigned long long len = ((st >= 1 && st <= nsteps) ? 1 : 0) + ((st + 1 < nsteps) ? ex->nranks : 0) +
                                           ((st >= ulag && st < nsteps + ulag) ? ex->nranks : 0);
            tickets += groups * len;
        }
        a.total_tickets = (unsigned)tickets;
        a.upd_lag = ex->upd_lag;
    }
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
        if (sgd->grad_scale) return fail(JABAS_EINVAL, "exchange: gradient-norm clipping (grad_scale) is not supported");
        if ((rc = jb_fill_sgd_hp(a.hp, groups, ngroups, sgd))) return rc;
        if (sgd->dynamic) {
            if (sgd->dynamic->kind != OPT_SGD) return fail(JABAS_EINVAL, "the dynamic block holds Adam hyper-parameters");
            a.dyn = sgd->dynamic->dev;
        }
    } else {
        if (!b.m || !b.v) return fail(JABAS_EINVAL, "exp_avg and exp_avg_sq buffers are required");
        if (adam->grad_scale) return fail(JABAS_EINVAL, "exchange: gradient-norm clipping (grad_scale) is not supported");
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
    if (bufs[0].Kg > kExMaxSlots) return fail(JABAS_EINVAL, "exchange: at most 8 VSW gradients per launch");
    // ring: one 4 KB slot per stream of the widest phase, as many stages as fit the budget
    const int slots = std::max(std::max(bufs[0].Kg, ex0->nranks), sgd ? 3 : 4);
    // Three resident CTAs per SM with a 64 KB ring each beat two with 96 KB on two GPUs (measured:
    // ResNet-50 layout 0.342 -> 0.318 ms, ViT-B/16 1.484 -> 1.426 ms, GNMT 2.158 -> 2.114 ms): more,
    // smaller items in flight shorten the tail and hide the per-item latencies better.  From four
    // GPUs on, where more of the traffic crosses NVLink, the deeper ring of the two-CTA form wins
    // (2^27 elements, 4 GPUs: 1.400 vs 1.435 ms), and so it does with more than five streams per stage.
    const bool three = ex0->ctas_per_sm == 3 ||
                       (ex0->ctas_per_sm == 0 && ex0->nranks == 2 && slots * 3 * (int)kTileBytes <= 64 * 1024);
    const int ring_budget = three ? 64 * 1024 : kRingBudgetBytes;
    ExKernel kern = three ? (sgd ? exchange_kernel<OPT_SGD, 3> : exchange_kernel<OPT_ADAM, 3>)
                          : (sgd ? exchange_kernel<OPT_SGD, 2> : exchange_kernel<OPT_ADAM, 2>);
    ExEmuKernel emu = three ? (sgd ? exchange_emu_kernel<OPT_SGD, 3> : exchange_emu_kernel<OPT_ADAM, 3>)
                            : (sgd ? exchange_emu_kernel<OPT_SGD, 2> : exchange_emu_kernel<OPT_ADAM, 2>);
    int stages = ring_budget / (slots * (int)kTileBytes);
    if (stages < 2) return fail(JABAS_EINVAL, "exchange: the ring holds fewer than two stages for this many streams");
    if (stages > kExMaxStages) stages = kExMaxStages;
    const size_t dyn_smem = (size_t)stages * slots * kTileBytes;
    jabas_ctx_t* ctx = ex0->ctx;
    int per_sm = 0;
    {
        const void* key = nlocal == 1 ? reinterpret_cast<const void*>(kern) : reinterpret_cast<const void*>(emu);
        std::lock_guard<std::mutex> lk(ctx->mu);
        auto it = ctx->occ.find(key);
        if (it != ctx->occ.end()) per_sm = it->second;
        if (per_sm == 0) {
            // occupancy for the full ring budget: the grid does not depend on the launch's stream count
            cudaError_t e = nlocal == 1
                ? cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_budget)
                : cudaFuncSetAttribute(emu, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_budget);
            if (e == cudaSuccess)
                e = nlocal == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kExThreads, ring_budget)
                                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, emu, kExThreads, ring_budget);
            if (e != cudaSuccess) return fail(JABAS_ECUDA, cudaGetErrorString(e));
            if (per_sm < 1) per_sm = 1;
            if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
            ctx->occ[key] = per_sm;
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (nlocal == 1) {
        ExArgs a;
        unsigned long long grid = (unsigned long long)ctx->sm_count * per_sm;
        if (ex0->grid_limit && grid > ex0->grid_limit) grid = ex0->grid_limit;
        if ((rc = fill_args(ex0, (unsigned)grid, bufs[0], a, n, base, slot_base, divisor, half_divisor, layout, groups, ngroups, sgd, adam)))
            return rc;
        if (grid > a.total_tickets) grid = a.total_tickets;
        a.ring_stages = stages; a.ring_slots = slots; a.opt = sgd ? OPT_SGD : OPT_ADAM;
        kern<<<(unsigned)grid, kExThreads, dyn_smem, st>>>(a);
        JB_CUDA(cudaGetLastError());
        return JABAS_OK;
    }
    // all ranks on this GPU, one launch: every CTA must be resident, because ranks wait on one another
    std::vector<ExArgs> h((size_t)nlocal);
    const unsigned gx = (unsigned)((ctx->sm_count * per_sm) / nlocal);
    if (gx < 1) return fail(JABAS_EINVAL, "exchange: the GPU cannot hold one CTA per rank");
    for (int r = 0; r < nlocal; ++r) {
        if (!exs[r] || exs[r]->ctx != ctx || exs[r]->nranks != nlocal || exs[r]->rank != r)
            return fail(JABAS_EINVAL, "exchange: the single-GPU form takes the ranks 0..n-1 of one context, in order");
        if (bufs[r].Kg != bufs[0].Kg) return fail(JABAS_EINVAL, "exchange: every rank must have the same number of VSWs here");
        if ((rc = fill_args(exs[r], gx, bufs[r], h[r], n, base, slot_base, divisor, half_divisor, layout, groups, ngroups, sgd, adam)))
            return rc;
        h[r].ring_stages = stages; h[r].ring_slots = slots; h[r].opt = sgd ? OPT_SGD : OPT_ADAM;
    }
    if (!ex0->d_emu) JB_CUDA(cudaMalloc(&ex0->d_emu, sizeof(ExArgs) * kExMaxRanks));
    JB_CUDA(cudaMemcpyAsync(ex0->d_emu, h.data(), sizeof(ExArgs) * nlocal, cudaMemcpyHostToDevice, st));
    JB_CUDA(cudaStreamSynchronize(st));          // h leaves scope; this form is for tests
    emu<<<dim3(gx, (unsigned)nlocal), kExThreads, dyn_smem, st>>>(ex0->d_emu);
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
