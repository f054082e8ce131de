// Multi-tensor fused optimizer steps, gradient norm / clipping and the
// inf/nan check of the loss scaler, as single launches over a table of tensors.
//
// The reference runs its optimizers on the host: a CUDA parameter is copied to
// the CPU, updated by hot::fused_adam_multi and copied back, four transfers per
// tensor per step (torch/optim/adam.h:192-220, 338-377).  Here one kernel
// launch updates every tensor of a parameter group in place; a table in device
// memory lists, per 64K-element chunk, the tensor it belongs to.
//
// Update rules follow the reference's files (torch/optim/{sgd,adam,rmsprop,
// lion,sophia,nadam,radam,adagrad,adadelta,adamax,asgd}.h).  Parameters and
// state are fp32; gradients may be fp32 or bf16; an optional bf16 copy of the
// parameter is written in the same pass (fp32 master weights, bf16 compute).
#include "common.cuh"

#include <algorithm>

namespace ptb {

constexpr int OPT_CHUNK = 65536;
constexpr int OPT_THREADS = 512;

enum OptKind : int {
    OPT_SGD = 0, OPT_ADAM = 1, OPT_ADAMW = 2, OPT_RMSPROP = 3, OPT_LION = 4, OPT_SOPHIA = 5, OPT_NADAM = 6,
    OPT_RADAM = 7, OPT_ADAGRAD = 8, OPT_ADADELTA = 9, OPT_ADAMAX = 10, OPT_ASGD = 11,
    OPT_LAMB = 12,          // three launches, see lamb_stage1_kernel
};

struct OptTensor {          // one row of the device-side table
    float* p;
    const void* g;
    float* s0;
    float* s1;
    float* s2;
    __nv_bfloat16* p_lowp;  // optional bf16 shadow of p
    long long numel;
};

struct OptArgs {
    const OptTensor* tensors;
    const int2* chunks;     // {tensor index, chunk index within the tensor}
    int kind;
    int grad_bf16;
    float h[16];            // hyper-parameters, meaning depends on `kind` (see apply())
    const float* grad_scale;   // optional device scalar multiplied into every gradient (clipping / unscaling)
    const int* skip;           // optional device flag: non-zero => leave everything untouched (inf/nan found)
};

template <bool BF16>
__device__ __forceinline__ float load_grad(const void* g, long long i) {
    if (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]);
    return reinterpret_cast<const float*>(g)[i];
}

// One element.  s0/s1/s2 are the state slots; returns the new parameter.
__device__ __forceinline__ float apply(int kind, const float* h, float p, float g, float& s0, float& s1, float& s2) {
    switch (kind) {
        case OPT_SGD: {
            // h: lr, momentum, dampening, weight_decay, nesterov, first_step
            const float lr = h[0], mom = h[1], damp = h[2], wd = h[3];
            if (wd != 0.f) g += wd * p;
            if (mom != 0.f) {
                s0 = (h[5] != 0.f) ? g : mom * s0 + (1.f - damp) * g;
                g = (h[4] != 0.f) ? g + mom * s0 : s0;
            }
            return p - lr * g;
        }
        case OPT_ADAM:
        case OPT_ADAMW: {
            // h: lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, amsgrad
            const float lr = h[0], b1 = h[1], b2 = h[2], eps = h[3], wd = h[4], bc1 = h[5], bc2 = h[6];
            if (kind == OPT_ADAMW) p *= 1.f - lr * wd;
            else if (wd != 0.f) g += wd * p;
            s0 = b1 * s0 + (1.f - b1) * g;
            s1 = b2 * s1 + (1.f - b2) * g * g;
            float v = s1;
            if (h[7] != 0.f) { s2 = fmaxf(s2, s1); v = s2; }
            const float denom = sqrtf(v) / sqrtf(bc2) + eps;
            return p - (lr / bc1) * s0 / denom;
        }
        case OPT_RMSPROP: {
            // h: lr, alpha, eps, weight_decay, momentum, centered
            const float lr = h[0], alpha = h[1], eps = h[2], wd = h[3], mom = h[4];
            if (wd != 0.f) g += wd * p;
            s0 = alpha * s0 + (1.f - alpha) * g * g;
            float avg;
            if (h[5] != 0.f) {
                s2 = alpha * s2 + (1.f - alpha) * g;
                avg = sqrtf(fmaxf(s0 - s2 * s2, 0.f)) + eps;
            } else {
                avg = sqrtf(s0) + eps;
            }
            if (mom > 0.f) {
                s1 = mom * s1 + g / avg;
                return p - lr * s1;
            }
            return p - lr * g / avg;
        }
        case OPT_LION: {
            // h: lr, beta1, beta2, weight_decay
            const float lr = h[0], b1 = h[1], b2 = h[2], wd = h[3];
            if (wd != 0.f) p *= 1.f - lr * wd;
            const float u = b1 * s0 + (1.f - b1) * g;
            p -= lr * ((u > 0.f) ? 1.f : (u < 0.f ? -1.f : 0.f));
            s0 = b2 * s0 + (1.f - b2) * g;
            return p;
        }
        case OPT_SOPHIA: {
            // h: lr, beta1, beta2, eps, weight_decay, rho
            const float lr = h[0], b1 = h[1], b2 = h[2], eps = h[3], wd = h[4], rho = h[5];
            if (wd != 0.f) p *= 1.f - lr * wd;
            s0 = b1 * s0 + (1.f - b1) * g;
            s1 = b2 * s1 + (1.f - b2) * g * g;
            const float r = fminf(fmaxf(s0 / fmaxf(s1, eps), -rho), rho);
            return p - lr * r;
        }
        case OPT_NADAM: {
            // h: lr, beta1, beta2, eps, weight_decay, mu_t, mu_next, mu_product, mu_product_next, bias_corr2
            const float lr = h[0], b1 = h[1], b2 = h[2], eps = h[3], wd = h[4];
            if (wd != 0.f) g += wd * p;
            s0 = b1 * s0 + (1.f - b1) * g;
            s1 = b2 * s1 + (1.f - b2) * g * g;
            const float denom = sqrtf(s1 / h[9]) + eps;
            p -= lr * (1.f - h[5]) / (1.f - h[7]) * g / denom;
            p -= lr * h[6] / (1.f - h[8]) * s0 / denom;
            return p;
        }
        case OPT_RADAM: {
            // h: lr, beta1, beta2, eps, weight_decay, bias_corr1, rect (0 => unrectified step), bias_corr2
            const float lr = h[0], b1 = h[1], b2 = h[2], eps = h[3], wd = h[4];
            if (wd != 0.f) g += wd * p;
            s0 = b1 * s0 + (1.f - b1) * g;
            s1 = b2 * s1 + (1.f - b2) * g * g;
            const float mhat = s0 / h[5];
            if (h[6] > 0.f) return p - lr * mhat * h[6] / (sqrtf(s1 / h[7]) + eps);
            return p - lr * mhat;
        }
        case OPT_ADAGRAD: {
            // h: clr (lr already decayed), eps, weight_decay
            if (h[2] != 0.f) g += h[2] * p;
            s0 += g * g;
            return p - h[0] * g / (sqrtf(s0) + h[1]);
        }
        case OPT_ADADELTA: {
            // h: lr, rho, eps, weight_decay
            const float rho = h[1], eps = h[2];
            if (h[3] != 0.f) g += h[3] * p;
            s0 = rho * s0 + (1.f - rho) * g * g;
            const float d = sqrtf(s1 + eps) / sqrtf(s0 + eps) * g;
            s1 = rho * s1 + (1.f - rho) * d * d;
            return p - h[0] * d;
        }
        case OPT_ADAMAX: {
            // h: lr, beta1, beta2, eps, weight_decay, bias_corr1
            const float b1 = h[1], b2 = h[2];
            if (h[4] != 0.f) g += h[4] * p;
            s0 = b1 * s0 + (1.f - b1) * g;
            s1 = fmaxf(b2 * s1, fabsf(g) + h[3]);
            return p - (h[0] / h[5]) * s0 / s1;
        }
        case OPT_ASGD: {
            // h: eta, lambd, weight_decay, mu ; s0 = averaged parameter
            if (h[2] != 0.f) g += h[2] * p;
            p *= 1.f - h[1] * h[0];
            p -= h[0] * g;
            s0 = (h[3] != 1.f) ? s0 + (p - s0) * h[3] : p;
            return p;
        }
    }
    return p;
}

template <bool BF16>
__global__ void __launch_bounds__(OPT_THREADS) multi_tensor_opt_kernel(const __grid_constant__ OptArgs A) {
    if (A.skip && *A.skip) return;
    const int2 ck = A.chunks[blockIdx.x];
    const OptTensor T = A.tensors[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    const float gs = A.grad_scale ? *A.grad_scale : 1.f;
    for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
        float p = T.p[i];
        const float g = load_grad<BF16>(T.g, i) * gs;
        float s0 = T.s0 ? T.s0[i] : 0.f, s1 = T.s1 ? T.s1[i] : 0.f, s2 = T.s2 ? T.s2[i] : 0.f;
        p = apply(A.kind, A.h, p, g, s0, s1, s2);
        T.p[i] = p;
        if (T.s0) T.s0[i] = s0;
        if (T.s1) T.s1[i] = s1;
        if (T.s2) T.s2[i] = s2;
        if (T.p_lowp) T.p_lowp[i] = __float2bfloat16_rn(p);
    }
}

// Sum of squares per chunk (+ inf/nan detection); a second tiny kernel folds the partials in a fixed
// order, so the norm is bitwise reproducible.
template <bool BF16>
__global__ void __launch_bounds__(OPT_THREADS) multi_tensor_sqnorm_kernel(const OptTensor* tensors, const int2* chunks,
                                                                        float* partial, int* found_inf) {
    __shared__ float red[OPT_THREADS / 32];
    const int2 ck = chunks[blockIdx.x];
    const OptTensor T = tensors[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    float s = 0.f;
    bool bad = false;
    for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
        const float g = load_grad<BF16>(T.g, i);
        bad |= !isfinite(g);
        s += g * g;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    if (bad && found_inf) atomicExch(found_inf, 1);
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < OPT_THREADS / 32 ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) partial[blockIdx.x] = t;
    }
}

// out[0] = total L2 norm, out[1] = clip coefficient min(1, max_norm / (norm + 1e-6)) * extra_scale
__global__ void finish_norm_kernel(const float* partial, int n, float max_norm, float extra_scale, float* out) {
    __shared__ float red[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) {
            const float norm = sqrtf(t);
            out[0] = norm;
            out[1] = (max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f) * extra_scale;
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(OPT_THREADS) multi_tensor_scale_kernel(const OptTensor* tensors, const int2* chunks,
                                                                       const float* scale) {
    const float s = *scale;
    if (s == 1.f) return;
    const int2 ck = chunks[blockIdx.x];
    const OptTensor T = tensors[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
        if (BF16) {
            __nv_bfloat16* g = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(T.g));
            g[i] = __float2bfloat16_rn(__bfloat162float(g[i]) * s);
        } else {
            float* g = reinterpret_cast<float*>(const_cast<void*>(T.g));
            g[i] *= s;
        }
    }
}

// ---- LAMB (torch/optim/lamb.h of the reference): the step size of a tensor is scaled by the trust ratio
// ||w|| / ||update||, a per-tensor quantity, so the step is three launches over the same table:
//   stage 1, per chunk: moments, the update direction u = m_hat / (sqrt(v_hat) + eps) + wd * w (kept in slot s2) and the
//            chunk's sums of w^2 and u^2;
//   stage 2, one warp per tensor: the partial sums of the tensor's chunks folded in a fixed order -> trust ratio;
//   stage 3, per chunk: w -= lr * trust * u (and the optional bf16 copy).
// h: lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2
template <bool BF16>
__global__ void __launch_bounds__(OPT_THREADS) lamb_stage1_kernel(const __grid_constant__ OptArgs A, float* __restrict__ partial) {
    __shared__ float red[2][OPT_THREADS / 32];
    if (A.skip && *A.skip) return;
    const int2 ck = A.chunks[blockIdx.x];
    const OptTensor T = A.tensors[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    const float gs = A.grad_scale ? *A.grad_scale : 1.f;
    const float b1 = A.h[1], b2 = A.h[2], eps = A.h[3], wd = A.h[4], bc1 = A.h[5], bc2 = A.h[6];
    float sw = 0.f, su = 0.f;
    for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
        const float p = T.p[i];
        const float g = load_grad<BF16>(T.g, i) * gs;
        const float m = b1 * T.s0[i] + (1.f - b1) * g;
        const float v = b2 * T.s1[i] + (1.f - b2) * g * g;
        T.s0[i] = m;
        T.s1[i] = v;
        const float u = (m / bc1) / (sqrtf(v / bc2) + eps) + wd * p;
        T.s2[i] = u;
        sw += p * p;
        su += u * u;
    }
    sw = warp_sum(sw);
    su = warp_sum(su);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = sw; red[1][threadIdx.x >> 5] = su; }
    __syncthreads();
    if (threadIdx.x < 32) {
        float a = threadIdx.x < OPT_THREADS / 32 ? red[0][threadIdx.x] : 0.f, b = threadIdx.x < OPT_THREADS / 32 ? red[1][threadIdx.x] : 0.f;
        a = warp_sum(a);
        b = warp_sum(b);
        if (threadIdx.x == 0) { partial[2 * blockIdx.x] = a; partial[2 * blockIdx.x + 1] = b; }
    }
}
// chunk_start[t] .. chunk_start[t+1]: the chunks of tensor t.  One warp per tensor.
__global__ void lamb_trust_kernel(const int* __restrict__ chunk_start, int n_tensors, const float* __restrict__ partial,
                                  float* __restrict__ trust, const int* skip) {
    if (skip && *skip) return;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tensors) return;
    float a = 0.f, b = 0.f;
    for (int c = chunk_start[t] + lane; c < chunk_start[t + 1]; c += 32) { a += partial[2 * c]; b += partial[2 * c + 1]; }
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) trust[t] = (a > 0.f && b > 0.f) ? sqrtf(a) / sqrtf(b) : 1.f;
}
__global__ void __launch_bounds__(OPT_THREADS) lamb_stage3_kernel(const __grid_constant__ OptArgs A, const float* __restrict__ trust) {
    if (A.skip && *A.skip) return;
    const int2 ck = A.chunks[blockIdx.x];
    const OptTensor T = A.tensors[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    const float step = A.h[0] * trust[ck.x];
    for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
        const float p = T.p[i] - step * T.s2[i];
        T.p[i] = p;
        if (T.p_lowp) T.p_lowp[i] = __float2bfloat16_rn(p);
    }
}

// ---- AdamKiller (torch/optim/adamkiller.h of the reference): gradient clipping per tensor, a momentum coefficient that
// follows the change of the gradient, a look-ahead on the gradient difference, a per-tensor step size from the ratio of
// weight and gradient norms, and a cap on the update norm.  Each of these is a per-tensor reduction feeding an
// element-wise pass, so the step is four element-wise launches over the group with a one-warp-per-tensor fold between
// them; nothing comes back to the host.
// Table A rows: s0 = m, s1 = v; table B rows (same order): s0 = previous gradient, s1 = gradient-difference average (or
// null), s2 = scratch (effective gradient, then the update).
// h: lr, beta1_min, beta1_max, beta2, eps, weight_decay, adaptive, per_layer, predict, restart, max_grad_norm,
//    lr_scale_min, lr_scale_max, step, has_prev
// per-tensor scalars ts[t][8]: 0 gradient scale, 1 beta1, 2 1 - beta1^t, 3 step size, 4 update clip
constexpr int AK_TS = 8;
struct Hyper16 { float v[16]; };

__device__ __forceinline__ void block_sums3(float a, float b, float c, float* out3) {
    __shared__ float red[3][OPT_THREADS / 32];
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a; red[1][threadIdx.x >> 5] = b; red[2][threadIdx.x >> 5] = c; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const bool in = threadIdx.x < OPT_THREADS / 32;
        a = warp_sum(in ? red[0][threadIdx.x] : 0.f);
        b = warp_sum(in ? red[1][threadIdx.x] : 0.f);
        c = warp_sum(in ? red[2][threadIdx.x] : 0.f);
        if (threadIdx.x == 0) { out3[0] = a; out3[1] = b; out3[2] = c; }
    }
}

template <bool BF16, int STAGE>
__global__ void __launch_bounds__(OPT_THREADS) adamkiller_pass_kernel(const __grid_constant__ OptArgs A, const OptTensor* __restrict__ tabB,
                                                                      float* __restrict__ partial, const float* __restrict__ ts) {
    if (A.skip && *A.skip) return;
    const int2 ck = A.chunks[blockIdx.x];
    const OptTensor T = A.tensors[ck.x];
    const OptTensor B = tabB[ck.x];
    const long long base = (long long)ck.y * OPT_CHUNK;
    const long long end = min(base + OPT_CHUNK, T.numel);
    const float gs = A.grad_scale ? *A.grad_scale : 1.f;
    const float* h = A.h;
    const bool has_prev = h[14] != 0.f;
    const float* my = ts + (size_t)ck.x * AK_TS;
    float a = 0.f, b = 0.f, c = 0.f;
    if (STAGE == 1) {                       // squared norm of the gradient
        for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) { const float g = load_grad<BF16>(T.g, i) * gs; a += g * g; }
    } else if (STAGE == 2) {                // clipped gradient, look-ahead, norms of the difference / the effective gradient / the weights
        const float gscale = my[0];
        const bool predict = h[8] != 0.f && has_prev && B.s1 != nullptr;
        for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
            const float sg = load_grad<BF16>(T.g, i) * gs * gscale;
            float eff = sg;
            if (has_prev) {
                const float d = sg - B.s0[i];
                a += d * d;
                if (predict) {
                    const float e = 0.5f * B.s1[i] + 0.5f * d;
                    B.s1[i] = e;
                    eff += 0.5f * e;
                }
            }
            B.s0[i] = sg;
            B.s2[i] = eff;
            b += eff * eff;
            const float p = T.p[i];
            c += p * p;
        }
    } else if (STAGE == 3) {                // moments and the update, its squared norm
        const float b1 = my[1], bc1 = my[2], step = my[3], b2 = h[3], eps = h[4];
        const float bc2 = 1.f - powf(b2, h[13]);
        for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
            const float eff = B.s2[i];
            const float m = b1 * T.s0[i] + (1.f - b1) * eff;
            const float v = b2 * T.s1[i] + (1.f - b2) * eff * eff;
            T.s0[i] = m;
            T.s1[i] = v;
            const float u = (m / bc1) / sqrtf(v / bc2 + eps) * step;
            B.s2[i] = u;
            a += u * u;
        }
    } else {                                // apply
        const float step = my[3], clip = my[4], wd = h[5];
        const float keep = wd > 0.f ? 1.f - step * wd : 1.f;
        const bool restart = h[9] != 0.f;
        for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
            const float p = T.p[i] * keep - B.s2[i] * clip;
            T.p[i] = p;
            if (T.p_lowp) T.p_lowp[i] = __float2bfloat16_rn(p);
            if (restart) T.s0[i] *= 0.1f;
        }
        return;
    }
    block_sums3(a, b, c, partial + 3 * (size_t)blockIdx.x);
}

// One warp per tensor folds the chunk partials of the pass before it (fixed order) into the per-tensor scalars.
template <int STAGE>
__global__ void adamkiller_fold_kernel(const int* __restrict__ chunk_start, int n_tensors, const float* __restrict__ partial,
                                       float* __restrict__ ts, const Hyper16 h16, const int* skip) {
    if (skip && *skip) return;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tensors) return;
    float a = 0.f, b = 0.f, c = 0.f;
    for (int k = chunk_start[t] + lane; k < chunk_start[t + 1]; k += 32) { a += partial[3 * k]; b += partial[3 * k + 1]; c += partial[3 * k + 2]; }
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    if (lane) return;
    float* my = ts + (size_t)t * AK_TS;
    const float* h = h16.v;
    const float lr = h[0];
    if (STAGE == 1) {
        const float gn = sqrtf(a), mx = h[10];
        my[0] = (gn > mx && gn > 1e-12f) ? mx / gn : 1.f;
    } else if (STAGE == 2) {
        const bool has_prev = h[14] != 0.f;
        float beta1 = h[2];
        if (h[6] != 0.f && has_prev) {
            const float curv = sqrtf(a) / (lr + 1e-12f);
            beta1 = h[2] - fminf(curv / 100.f, 1.f) * (h[2] - h[1]);
            beta1 = fmaxf(h[1], fminf(h[2], beta1));
        }
        my[1] = beta1;
        my[2] = 1.f - powf(beta1, h[13]);
        float step = lr;
        if (h[7] != 0.f) {
            const float en = sqrtf(b), wn = sqrtf(c);
            if (en > 1e-8f && wn > 1e-8f) step = lr * fmaxf(h[11], fminf(h[12], wn / (en + h[5] * wn)));
        }
        my[3] = step;
    } else {
        const float un = sqrtf(a), cap = 2.f * my[3];
        my[4] = (un > cap && un > 1e-12f) ? cap / un : 1.f;
    }
}

// ---- Adafactor (torch/optim/adafactor.h of the reference): the second moment of a matrix is kept as a row vector and a
// column vector.  Per tensor: row sums (+ the weight norm), column sums in row splits, a fold that advances both vectors and
// derives the step size, a pass for the norm of the update, and the apply pass, which recomputes the update instead of
// storing it.  h: lr_base (relative or fixed), eps1, eps2, clip_threshold, beta2_t, beta1, weight_decay, scale_parameter
// ts[8]: 0 sum p^2, 1 mean of the row vector, 2 step size, 3 1 / clip scale
constexpr int AF_SPLIT_ROWS = 256;

template <bool BF16>
__global__ void __launch_bounds__(256) adafactor_rows_kernel(const float* __restrict__ p, const void* __restrict__ g, int rows, int cols,
                                                             const float* gsp, const int* skip, float eps1, float* __restrict__ rowsum,
                                                             float* __restrict__ psq_part) {
    // one warp per row (grid-stride): sum of g^2 + eps1 over the row, and this block's share of sum p^2
    if (skip && *skip) return;
    const float gs = gsp ? *gsp : 1.f;
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float psq = 0.f;
    for (int r = blockIdx.x * nw + wib; r < rows; r += gridDim.x * nw) {
        float a = 0.f;
        for (int c = lane; c < cols; c += 32) {
            const long long i = (long long)r * cols + c;
            const float gv = load_grad<BF16>(g, i) * gs;
            a += gv * gv + eps1;
            const float pv = p[i];
            psq += pv * pv;
        }
        a = warp_sum(a);
        if (lane == 0) rowsum[r] = a;
    }
    __shared__ float red[8];
    psq = warp_sum(psq);
    if (lane == 0) red[wib] = psq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < nw; ++w) t += red[w];
        psq_part[blockIdx.x] = t;
    }
}
template <bool BF16>
__global__ void __launch_bounds__(256) adafactor_cols_kernel(const void* __restrict__ g, int rows, int cols, const float* gsp,
                                                             const int* skip, float eps1, float* __restrict__ colpart) {
    // grid (col blocks, row splits): one thread per column sums its column over the rows of the split
    if (skip && *skip) return;
    const float gs = gsp ? *gsp : 1.f;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.y * AF_SPLIT_ROWS, r1 = min(rows, r0 + AF_SPLIT_ROWS);
    float a = 0.f;
    for (int r = r0; r < r1; ++r) {
        const float gv = load_grad<BF16>(g, (long long)r * cols + c) * gs;
        a += gv * gv + eps1;
    }
    colpart[(size_t)blockIdx.y * cols + c] = a;
}
// One block: advance the row and column vectors (or nothing for a vector parameter), their mean, the step size.
__global__ void __launch_bounds__(1024) adafactor_fold_kernel(float* __restrict__ R, float* __restrict__ Cv, const float* __restrict__ rowsum,
                                                              const float* __restrict__ colpart, int rows, int cols, int nsplit,
                                                              const float* __restrict__ psq_part, int n_psq, long long numel,
                                                              Hyper16 H, float* __restrict__ ts, const int* skip) {
    __shared__ float red[32];
    if (skip && *skip) return;
    const float* h = H.v;
    const float b2 = h[4];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    auto block_sum = [&](float v) -> float {
        v = warp_sum(v);
        __syncthreads();
        if (lane == 0) red[wib] = v;
        __syncthreads();
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        return t;
    };
    float a = 0.f;
    for (int i = threadIdx.x; i < n_psq; i += blockDim.x) a += psq_part[i];
    const float psq = block_sum(a);
    float rsum = 0.f;
    if (R) {
        for (int r = threadIdx.x; r < rows; r += blockDim.x) {
            const float v = b2 * R[r] + (1.f - b2) * rowsum[r] / (float)cols;
            R[r] = v;
            rsum += v;
        }
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            float t = 0.f;
            for (int k = 0; k < nsplit; ++k) t += colpart[(size_t)k * cols + c];
            Cv[c] = b2 * Cv[c] + (1.f - b2) * t / (float)rows;
        }
    }
    const float rmean = block_sum(rsum) / (float)max(rows, 1);
    if (threadIdx.x == 0) {
        ts[0] = psq;
        ts[1] = rmean;
        float lr = h[0];
        if (h[7] != 0.f) lr *= fmaxf(h[2], sqrtf(psq / (float)max(numel, 1LL)));
        ts[2] = lr;
    }
}
// The update of element (r, c).  Factored: g / max(sqrt(R[r] / max(mean R, eps1) * C[c]), eps1); a vector parameter
// advances its full second moment here when `advance` is set (the apply pass) and reads the advanced value otherwise.
template <bool BF16>
__device__ __forceinline__ float adafactor_update(const void* g, long long i, int r, int c, float gs, const float* R, const float* Cv,
                                                  float* V, float rmean, float eps1, float b2, bool advance) {
    const float gv = load_grad<BF16>(g, i) * gs;
    float v;
    if (R) {
        v = R[r] / fmaxf(rmean, eps1) * Cv[c];
    } else {
        v = b2 * V[i] + (1.f - b2) * (gv * gv + eps1);
        if (advance) V[i] = v;
    }
    return gv / fmaxf(sqrtf(v), eps1);
}
template <bool BF16, bool APPLY>
__global__ void __launch_bounds__(256) adafactor_update_kernel(float* __restrict__ p, const void* __restrict__ g, const float* __restrict__ R,
                                                               const float* __restrict__ Cv, float* __restrict__ V, float* __restrict__ mom,
                                                               __nv_bfloat16* __restrict__ lowp, int rows, int cols, const float* gsp,
                                                               const int* skip, Hyper16 H, const float* __restrict__ ts,
                                                               float* __restrict__ part) {
    if (skip && *skip) return;
    const float gs = gsp ? *gsp : 1.f;
    const float* h = H.v;
    const float eps1 = h[1], b2 = h[4], rmean = ts[1];
    const long long n = (long long)rows * cols;
    float a = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
        float u = adafactor_update<BF16>(g, i, r, c, gs, R, Cv, V, rmean, eps1, b2, APPLY);
        if (!APPLY) { a += u * u; continue; }
        u *= ts[3];
        if (mom) {
            const float m = h[5] * mom[i] + (1.f - h[5]) * u;
            mom[i] = m;
            u = m;
        }
        const float lr = ts[2];
        float pv = p[i];
        if (h[6] != 0.f) pv *= 1.f - lr * h[6];
        pv -= lr * u;
        p[i] = pv;
        if (lowp) lowp[i] = __float2bfloat16_rn(pv);
    }
    if (APPLY) return;
    __shared__ float red[8];
    a = warp_sum(a);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += red[w];
        part[blockIdx.x] = t;
    }
}
__global__ void adafactor_clip_kernel(const float* __restrict__ part, int n, long long numel, float clip_threshold, float* __restrict__ ts,
                                      const int* skip) {
    if (skip && *skip) return;
    float a = 0.f;
    for (int i = threadIdx.x; i < n; i += 32) a += part[i];
    a = warp_sum(a);
    if (threadIdx.x == 0) ts[3] = 1.f / fmaxf(1.f, sqrtf(a / (float)max(numel, 1LL)) / clip_threshold);
}

}  // namespace ptb

using namespace ptb;

// Fused AdamKiller step over one parameter group.  tensors / tensors_b: the two tables (see above), same row order;
// partial: 3 * n_chunks floats; ts: 8 * n_tensors floats (readable afterwards: scale, beta1, 1 - beta1^t, step size, clip).
PTB_API int ptb_multi_tensor_adamkiller(const void* tensors, const void* tensors_b, const void* chunks, int n_chunks,
                                        const int* chunk_start, int n_tensors, int grad_bf16, const float* h,
                                        const float* grad_scale, const int* skip, float* partial, float* ts, cudaStream_t stream) {
    if (n_chunks <= 0) return 0;
    OptArgs a;
    a.tensors = (const OptTensor*)tensors;
    a.chunks = (const int2*)chunks;
    a.kind = 13;
    a.grad_bf16 = grad_bf16;
    for (int i = 0; i < 16; ++i) a.h[i] = h[i];
    a.grad_scale = grad_scale;
    a.skip = skip;
    const OptTensor* tb = (const OptTensor*)tensors_b;
    const int fold_blocks = (n_tensors + 7) / 8;
    Hyper16 h_dev;
    for (int i = 0; i < 16; ++i) h_dev.v[i] = h[i];
#define AK_PASS(S)                                                                                                      \
    do {                                                                                                                \
        if (grad_bf16) adamkiller_pass_kernel<true, S><<<n_chunks, OPT_THREADS, 0, stream>>>(a, tb, partial, ts);        \
        else adamkiller_pass_kernel<false, S><<<n_chunks, OPT_THREADS, 0, stream>>>(a, tb, partial, ts);                 \
    } while (0)
    AK_PASS(1);
    adamkiller_fold_kernel<1><<<fold_blocks, 256, 0, stream>>>(chunk_start, n_tensors, partial, ts, h_dev, skip);
    AK_PASS(2);
    adamkiller_fold_kernel<2><<<fold_blocks, 256, 0, stream>>>(chunk_start, n_tensors, partial, ts, h_dev, skip);
    AK_PASS(3);
    adamkiller_fold_kernel<3><<<fold_blocks, 256, 0, stream>>>(chunk_start, n_tensors, partial, ts, h_dev, skip);
    AK_PASS(4);
#undef AK_PASS
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Fused Adafactor step of ONE parameter.  rows x cols: the matrix (rows = 1 for a vector, which keeps a full second moment in
// V and passes R = C = null).  scratch: rows + ceil(rows / 256) * cols + 2 * blocks floats with blocks = 592; ts: 8 floats.
PTB_API int ptb_adafactor_step(float* p, const void* g, int grad_bf16, float* R, float* Cv, float* V, float* mom, void* lowp, int rows,
                               int cols, const float* h, const float* grad_scale, const int* skip, float* scratch, float* ts,
                               cudaStream_t stream) {
    const long long numel = (long long)rows * cols;
    if (numel <= 0) return 0;
    Hyper16 H;
    for (int i = 0; i < 16; ++i) H.v[i] = h[i];
    const int blocks = 592;
    const int nsplit = (rows + AF_SPLIT_ROWS - 1) / AF_SPLIT_ROWS;
    float* rowsum = scratch;
    float* colpart = rowsum + rows;
    float* psq_part = colpart + (size_t)nsplit * cols;
    float* upd_part = psq_part + blocks;
    const int row_blocks = std::min(blocks, (rows + 7) / 8);
    if (grad_bf16) adafactor_rows_kernel<true><<<row_blocks, 256, 0, stream>>>(p, g, rows, cols, grad_scale, skip, h[1], rowsum, psq_part);
    else adafactor_rows_kernel<false><<<row_blocks, 256, 0, stream>>>(p, g, rows, cols, grad_scale, skip, h[1], rowsum, psq_part);
    if (R) {
        const dim3 grid((cols + 255) / 256, nsplit);
        if (grad_bf16) adafactor_cols_kernel<true><<<grid, 256, 0, stream>>>(g, rows, cols, grad_scale, skip, h[1], colpart);
        else adafactor_cols_kernel<false><<<grid, 256, 0, stream>>>(g, rows, cols, grad_scale, skip, h[1], colpart);
    }
    adafactor_fold_kernel<<<1, 1024, 0, stream>>>(R, Cv, rowsum, colpart, rows, cols, nsplit, psq_part, row_blocks, numel, H, ts, skip);
    const int ub = (int)std::min<long long>(blocks, (numel + 255) / 256);
    __nv_bfloat16* lp = (__nv_bfloat16*)lowp;
    if (grad_bf16) adafactor_update_kernel<true, false><<<ub, 256, 0, stream>>>(p, g, R, Cv, V, mom, lp, rows, cols, grad_scale, skip, H, ts, upd_part);
    else adafactor_update_kernel<false, false><<<ub, 256, 0, stream>>>(p, g, R, Cv, V, mom, lp, rows, cols, grad_scale, skip, H, ts, upd_part);
    adafactor_clip_kernel<<<1, 32, 0, stream>>>(upd_part, ub, numel, h[3], ts, skip);
    if (grad_bf16) adafactor_update_kernel<true, true><<<ub, 256, 0, stream>>>(p, g, R, Cv, V, mom, lp, rows, cols, grad_scale, skip, H, ts, upd_part);
    else adafactor_update_kernel<false, true><<<ub, 256, 0, stream>>>(p, g, R, Cv, V, mom, lp, rows, cols, grad_scale, skip, H, ts, upd_part);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Fused LAMB step.  chunk_start: device int [n_tensors + 1] (prefix sums of the chunk counts, in table order);
// partial: 2 * n_chunks floats of scratch; trust: n_tensors floats (the trust ratios of this step, readable afterwards).
// Every row of the table needs all three state slots (moments and the update buffer).
PTB_API int ptb_multi_tensor_lamb(const void* tensors, const void* chunks, int n_chunks, const int* chunk_start, int n_tensors,
                                  int grad_bf16, const float* h, const float* grad_scale, const int* skip, float* partial,
                                  float* trust, cudaStream_t stream) {
    if (n_chunks <= 0) return 0;
    OptArgs a;
    a.tensors = (const OptTensor*)tensors;
    a.chunks = (const int2*)chunks;
    a.kind = OPT_LAMB;
    a.grad_bf16 = grad_bf16;
    for (int i = 0; i < 16; ++i) a.h[i] = h[i];
    a.grad_scale = grad_scale;
    a.skip = skip;
    if (grad_bf16) lamb_stage1_kernel<true><<<n_chunks, OPT_THREADS, 0, stream>>>(a, partial);
    else lamb_stage1_kernel<false><<<n_chunks, OPT_THREADS, 0, stream>>>(a, partial);
    lamb_trust_kernel<<<(n_tensors + 7) / 8, 256, 0, stream>>>(chunk_start, n_tensors, partial, trust, skip);
    lamb_stage3_kernel<<<n_chunks, OPT_THREADS, 0, stream>>>(a, trust);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_opt_chunk() { return OPT_CHUNK; }
PTB_API int ptb_opt_tensor_bytes() { return (int)sizeof(OptTensor); }

// tensors: device array of OptTensor rows; chunks: device int2 array of n_chunks entries; h: 16 host floats.
PTB_API int ptb_multi_tensor_opt(const void* tensors, const void* chunks, int n_chunks, int kind, int grad_bf16,
                                 const float* h, const float* grad_scale, const int* skip, cudaStream_t stream) {
    if (n_chunks <= 0) return 0;
    OptArgs a;
    a.tensors = (const OptTensor*)tensors;
    a.chunks = (const int2*)chunks;
    a.kind = kind;
    a.grad_bf16 = grad_bf16;
    for (int i = 0; i < 16; ++i) a.h[i] = h[i];
    a.grad_scale = grad_scale;
    a.skip = skip;
    if (grad_bf16) multi_tensor_opt_kernel<true><<<n_chunks, OPT_THREADS, 0, stream>>>(a);
    else multi_tensor_opt_kernel<false><<<n_chunks, OPT_THREADS, 0, stream>>>(a);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Total gradient norm into out[0], clip coefficient into out[1]; found_inf (optional) is set to 1 if any
// gradient is inf/nan.  `partial` holds n_chunks floats of scratch.
PTB_API int ptb_multi_tensor_grad_norm(const void* tensors, const void* chunks, int n_chunks, int grad_bf16, float* partial,
                                       float max_norm, float extra_scale, float* out, int* found_inf, cudaStream_t stream) {
    if (n_chunks > 0) {
        if (grad_bf16) multi_tensor_sqnorm_kernel<true><<<n_chunks, OPT_THREADS, 0, stream>>>((const OptTensor*)tensors, (const int2*)chunks, partial, found_inf);
        else multi_tensor_sqnorm_kernel<false><<<n_chunks, OPT_THREADS, 0, stream>>>((const OptTensor*)tensors, (const int2*)chunks, partial, found_inf);
    }
    finish_norm_kernel<<<1, 1024, 0, stream>>>(partial, n_chunks, max_norm, extra_scale, out);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_multi_tensor_scale(const void* tensors, const void* chunks, int n_chunks, int grad_bf16, const float* scale,
                                   cudaStream_t stream) {
    if (n_chunks <= 0) return 0;
    if (grad_bf16) multi_tensor_scale_kernel<true><<<n_chunks, OPT_THREADS, 0, stream>>>((const OptTensor*)tensors, (const int2*)chunks, scale);
    else multi_tensor_scale_kernel<false><<<n_chunks, OPT_THREADS, 0, stream>>>((const OptTensor*)tensors, (const int2*)chunks, scale);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
