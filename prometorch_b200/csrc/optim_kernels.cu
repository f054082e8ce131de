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

}  // namespace ptb

using namespace ptb;

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
