/*
 * TEST INFRASTRUCTURE — CPU oracle for the JABAS/IIDP per-iteration gradient path.
 *
 * This file is the checker, never the product: only tests, the smoke check and the
 * benchmark's CPU-baseline leg may load it.  The shipped library never links it.
 *
 * It restates, element by element and with every fp32 rounding written out, the
 * arithmetic that the reference executes through stock PyTorch ops on the path
 *
 *   K-VSW local aggregation -> bucket allreduce -> two-half cosine statistic
 *   -> SGD-momentum / Adam / AdamW update -> weight write-back to the K replicas.
 *
 * PARITY UNPINNED for the arithmetic in this file: the reference ships no tests,
 * golden vectors or known-answer fixtures, and the code that owns this arithmetic
 * (the IIDP submodule, IIDP's patch to PyTorch v1.8.1, torch.optim of v1.8.1) is
 * absent from the reference tree (.gitmodules:1-3, README.md:64-80).  The formulas
 * below are the published PyTorch v1.8.1 algorithms (torch/optim/_functional.py
 * `sgd`, `adam`, `adamw`; ATen `cosine_similarity`) as reached from the reference's
 * call sites, each cited beside the function.  The oracle is cross-checked against
 * the installed torch.optim on CPU by the test-suite.
 *
 * Rounding contract.  A PyTorch op of the form  a + alpha*b  (add with alpha,
 * addcmul, addcdiv) is one fused multiply-add on the reference's device kernels;
 * two separate ops (mul_ then add_) round twice.  This file is compiled with
 * -ffp-contract=off so that ONLY the fmaf() calls written here fuse.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* Local aggregation of the K virtual-stream-worker gradient buckets on one GPU into
 * the main replica's bucket.  The reference gives only VSW 0 a communicating hook
 * (jabas/train/trainer.py:461-468) and averages over T = total_num_decoupled_workers
 * (jabas/train/trainer.py:452-455); the summation itself lives in the absent IIDP
 * reducer, so its order is fixed here: ascending k in fp32, then one true division.
 *   half_out (nullable) receives the UNDIVIDED sum: the tensor that
 *   jabas/ddp_comm_hooks/similarity_allreduce.py:28 clones before the world allreduce.
 *   out may alias grads[0]. */
ORACLE_API void oracle_vsw_aggregate_f32(const float* const* grads, int K, float* out,
                                         float* half_out, size_t n, float divisor)
{
    for (size_t i = 0; i < n; ++i) {
        float s = grads[0][i];
        for (int k = 1; k < K; ++k) s = s + grads[k][i];
        if (half_out) half_out[i] = s;
        out[i] = s / divisor;
    }
}

/* In-place division of a bucket by a scalar: the `div_(T/2)` of
 * jabas/ddp_comm_hooks/similarity_allreduce.py:32 and the `div_(T)` of the world hook. */
ORACLE_API void oracle_div_f32(float* x, size_t n, float divisor)
{
    for (size_t i = 0; i < n; ++i) x[i] = x[i] / divisor;
}

/* stat[0] += <a,b>, stat[1] += |a|^2, stat[2] += |b|^2, products and sums in fp64.
 * These are the three reductions of ATen cosine_similarity as called at
 * jabas/train/trainer.py:478 (w12, w1, w2). */
ORACLE_API void oracle_dot_norms_f32(const float* a, const float* b, size_t n, double* stat)
{
    double d = 0.0, na = 0.0, nb = 0.0;
    for (size_t i = 0; i < n; ++i) {
        double x = (double)a[i], y = (double)b[i];
        d += x * y; na += x * x; nb += y * y;
    }
    stat[0] += d; stat[1] += na; stat[2] += nb;
}

/* The two-half statistic without the pair exchange: a rank holds the world mean g
 * and the mean `e` of its own parity sub-group (jabas/ddp_comm_hooks/
 * similarity_allreduce.py:28-33: clone, sub-group SUM, div_(T/2)).  With both
 * sub-groups of size T/2 the other half is o = 2g - e.  `half` is the sub-group SUM
 * (not yet divided); half_divisor = T/2. */
ORACLE_API void oracle_half_stat_f32(const float* g, const float* half, size_t n,
                                     float half_divisor, double* stat)
{
    double d = 0.0, ne = 0.0, no = 0.0;
    for (size_t i = 0; i < n; ++i) {
        float e = half[i] / half_divisor;
        float o = fmaf(2.0f, g[i], -e);
        double x = (double)e, y = (double)o;
        d += x * y; ne += x * x; no += y * y;
    }
    stat[0] += d; stat[1] += ne; stat[2] += no;
}

/* Single-GPU form of the statistic (an extension: the reference asserts an even
 * world size, jabas/train/trainer.py:430).  The halves are the VSWs of even and of
 * odd index on this GPU: E = (g_0 + g_2 + ...) / hd, O = (g_1 + g_3 + ...) / hd,
 * each summed in ascending k. */
ORACLE_API void oracle_vsw_parity_stat_f32(const float* const* grads, int K, size_t n,
                                           float half_divisor, double* stat)
{
    double d = 0.0, ne = 0.0, no = 0.0;
    for (size_t i = 0; i < n; ++i) {
        float e = grads[0][i], o = 0.0f;
        if (K > 1) o = grads[1][i];
        for (int k = 2; k < K; ++k) {
            if (k & 1) o = o + grads[k][i]; else e = e + grads[k][i];
        }
        e = e / half_divisor; o = o / half_divisor;
        double x = (double)e, y = (double)o;
        d += x * y; ne += x * x; no += y * y;
    }
    stat[0] += d; stat[1] += ne; stat[2] += no;
}

/* cos = w12 / sqrt(max(w1*w2, eps^2)) — ATen cosine_similarity of PyTorch v1.8.1
 * (the version the reference pins, README.md:66), called with the default eps=1e-8
 * at jabas/train/trainer.py:478.  Evaluated in fp64 on the fp64 sums, returned as fp32. */
ORACLE_API float oracle_cosine_from_stat(const double* stat, double eps)
{
    double den = stat[1] * stat[2];
    if (den < eps * eps) den = eps * eps;
    return (float)(stat[0] / sqrt(den));
}

/* torch.optim.SGD of v1.8.1 (torch/optim/_functional.py `sgd`), reached from
 * examples/resnet50/main.py:351-359:
 *   d = g + wd*p              (add with alpha: one fma; skipped when wd == 0)
 *   first step:  m = d        (clone)
 *   else:        m = mu*m     (mul_)  ;  m = m + (1-dampening)*d   (add_ with alpha: fma)
 *   nesterov:    d = d + mu*m (fma)   else d = m
 *   p = p + (-lr)*d           (add_ with alpha: fma)
 * Scalars arrive as fp64 (Python floats) and are rounded to fp32 once. */
ORACLE_API void oracle_sgd_momentum_f32(const float* g, float* p, float* m, size_t n,
                                        double lr, double weight_decay, double momentum,
                                        double dampening, int nesterov, int first_step)
{
    const float wd = (float)weight_decay, mu = (float)momentum;
    const float omd = (float)(1.0 - dampening), nlr = (float)(-lr);
    for (size_t i = 0; i < n; ++i) {
        float d = g[i];
        if (weight_decay != 0.0) d = fmaf(wd, p[i], d);
        if (momentum != 0.0) {
            float b;
            if (first_step) b = d;
            else { b = mu * m[i]; b = fmaf(omd, d, b); }
            m[i] = b;
            d = nesterov ? fmaf(mu, b, d) : b;
        }
        p[i] = fmaf(nlr, d, p[i]);
    }
}

/* torch.optim.Adam / AdamW of v1.8.1 (torch/optim/_functional.py `adam`, `adamw`),
 * reached from examples/vit/main.py:433-437 (AdamW), examples/gnmt/train.py:786-792
 * (Adam) and, argument for argument, examples/gnmt/seq2seq/train/shard_optimizer.py:77-90:
 *   decoupled:  p = p * (1 - lr*wd)                (mul_; scalar formed in fp64)
 *   coupled:    g = g + wd*p                       (fma; skipped when wd == 0)
 *   m = beta1*m (mul_) ; m = m + (1-beta1)*g       (fma)
 *   v = beta2*v (mul_) ; v = v + ((1-beta2)*g)*g   (addcmul: one mul, one fma)
 *   denom = sqrt(v) / sqrt(1-beta2^t) + eps        (three ops, three roundings)
 *   p = p + (-(lr/(1-beta1^t))) * (m/denom)        (addcdiv: one div, one fma)
 * `step` is the value AFTER the increment of shard_optimizer.py:70. */
ORACLE_API void oracle_adam_f32(const float* g, float* p, float* m, float* v, size_t n,
                                double lr, double weight_decay, double beta1, double beta2,
                                double eps, long long step, int decoupled)
{
    const double bc1 = 1.0 - pow(beta1, (double)step);
    const double bc2 = 1.0 - pow(beta2, (double)step);
    const float b1 = (float)beta1, b2 = (float)beta2;
    const float omb1 = (float)(1.0 - beta1), omb2 = (float)(1.0 - beta2);
    const float bc2s = (float)sqrt(bc2), epsf = (float)eps;
    const float nstep = (float)(-(lr / bc1));
    const float wd = (float)weight_decay;
    const float decay = (float)(1.0 - lr * weight_decay);
    for (size_t i = 0; i < n; ++i) {
        float gi = g[i], pi = p[i];
        if (decoupled) pi = pi * decay;
        else if (weight_decay != 0.0) gi = fmaf(wd, pi, gi);
        float mi = b1 * m[i];
        mi = fmaf(omb1, gi, mi);
        float vi = b2 * v[i];
        vi = fmaf(omb2 * gi, gi, vi);
        float denom = sqrtf(vi) / bc2s;
        denom = denom + epsf;
        pi = fmaf(nstep, mi / denom, pi);
        m[i] = mi; v[i] = vi; p[i] = pi;
    }
}

/* Weight write-back main replica -> VSW replicas 1..K-1: the per-parameter
 * dst.data.copy_(src.data) idiom of jabas/train/trainer.py:530-534; a bit copy. */
ORACLE_API void oracle_replicate_f32(const float* src, float* const* dst, int ndst, size_t n)
{
    for (int k = 0; k < ndst; ++k)
        if (dst[k] != src) memcpy(dst[k], src, n * sizeof(float));
}

/* Sum of squares in fp64 (gradient-norm clipping of
 * examples/gnmt/seq2seq/train/shard_optimizer.py:75-76). */
ORACLE_API double oracle_sumsq_f32(const float* x, size_t n)
{
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += (double)x[i] * (double)x[i];
    return s;
}

/* torch.nn.utils.clip_grad_norm_ of PyTorch v1.8.1 (norm_type 2), as reached from
 * examples/gnmt/seq2seq/train/trainer.py:157-161 and, per bucket, from
 * clip_grad_norm_for_overlap at examples/gnmt/seq2seq/train/shard_optimizer.py:75-76:
 *   total_norm = sqrt(sum g^2)  (here from the fp64 sum, rounded to fp32)
 *   clip_coef  = max_norm / (total_norm + 1e-6)              (fp32)
 *   if clip_coef < 1:  g = g * clip_coef                      (mul_)
 * Returns the coefficient; *norm_out (nullable) receives total_norm. */
ORACLE_API float oracle_clip_grad_norm_f32(float* g, size_t n, double max_norm, float* norm_out)
{
    const float total = (float)sqrt(oracle_sumsq_f32(g, n));
    const float coef = (float)max_norm / (total + 1e-6f);
    if (norm_out) *norm_out = total;
    if (coef < 1.0f)
        for (size_t i = 0; i < n; ++i) g[i] = g[i] * coef;
    return coef;
}
