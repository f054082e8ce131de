// Bandwidth-bound training kernels: RMSNorm forward/backward, rotary embedding
// forward/backward, SiLU/GELU-gated MLP activation forward/backward, and the
// fused softmax + cross-entropy (loss and gradient in one pass over the logits).
//
// The reference computes these with one thread per row and serial loops over
// the feature dimension (softmax_kernel, aten/src/ATen/cuda/CUDAKernels.cu:522-552;
// cross_entropy_loss_kernel, CUDAReduce.cu:606-683; rms_norm_kernel,
// CUDAInference.cu:19-76).  Here every kernel moves 16 bytes per thread per
// access, keeps a row in registers between its reduction and its update, and
// touches HBM once per operand.
#include "common.cuh"

namespace ptb {

template <typename T> struct Vec8;                      // 8 elements = one 16-byte (bf16) or two 16-byte (fp32) accesses
template <> struct Vec8<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
    __device__ __forceinline__ void get(float* f) const {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
    __device__ __forceinline__ void set(const float* f) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    }
};
template <> struct Vec8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = reinterpret_cast<const float4*>(p)[0]; b = reinterpret_cast<const float4*>(p)[1]; }
    __device__ __forceinline__ void store(float* p) const { reinterpret_cast<float4*>(p)[0] = a; reinterpret_cast<float4*>(p)[1] = b; }
    __device__ __forceinline__ void get(float* f) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w; }
    __device__ __forceinline__ void set(const float* f) { a = make_float4(f[0], f[1], f[2], f[3]); b = make_float4(f[4], f[5], f[6], f[7]); }
};

__device__ __forceinline__ float block_reduce_sum(float v, float* sm) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sm[w] = v;
    __syncthreads();
    float t = l < nw ? sm[l] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_reduce_max(float v, float* sm) {
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sm[w] = v;
    __syncthreads();
    float t = l < nw ? sm[l] : -INFINITY;
    return warp_max(t);
}

// ------------------------------------------------------------------------------------------ RMSNorm
constexpr int RMS_MAXV = 4;      // 8-element vectors per thread: H <= 8 * RMS_MAXV * blockDim

template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, float* __restrict__ rstd,
                                   int H, float eps, const T* __restrict__ resid_in, T* __restrict__ resid_out) {
    // optional fused residual add: h = x + resid_in is written to resid_out and normalised
    __shared__ float sm[32];
    const size_t row = blockIdx.x;
    const int nv = H / 8;
    float v[RMS_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < RMS_MAXV; ++k) {
        const int i = k * blockDim.x + threadIdx.x;
        if (i < nv) {
            Vec8<T> t;
            t.load(x + row * H + (size_t)i * 8);
            t.get(v[k]);
            if (resid_in) {
                Vec8<T> r;
                float rf[8];
                r.load(resid_in + row * H + (size_t)i * 8);
                r.get(rf);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[k][j] += rf[j];
                Vec8<T> o;
                o.set(v[k]);
                o.get(v[k]);            // normalise what was actually stored (rounded to T)
                o.store(resid_out + row * H + (size_t)i * 8);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
        }
    }
    ss = block_reduce_sum(ss, sm);
    const float rs = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = rs;
#pragma unroll
    for (int k = 0; k < RMS_MAXV; ++k) {
        const int i = k * blockDim.x + threadIdx.x;
        if (i < nv) {
            Vec8<T> wv, o;
            float wf[8], of[8];
            wv.load(w + (size_t)i * 8);
            wv.get(wf);
#pragma unroll
            for (int j = 0; j < 8; ++j) of[j] = v[k][j] * rs * wf[j];
            o.set(of);
            o.store(y + row * H + (size_t)i * 8);
        }
    }
}

// dx = rstd * (w*dy) - x * rstd^3 * mean(w*dy*x); per-CTA partial dw[H] over the CTA's rows.
template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                                   const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                                   int H, const T* __restrict__ dresid) {
    // dresid (optional): gradient flowing into the residual stream output, added to dx
    __shared__ float sm[32];
    const int nv = H / 8;
    float wf[RMS_MAXV][8], dwacc[RMS_MAXV][8];
#pragma unroll
    for (int k = 0; k < RMS_MAXV; ++k) {
        const int i = k * blockDim.x + threadIdx.x;
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[k][j] = 0.f;
        if (i < nv) { Vec8<T> t; t.load(w + (size_t)i * 8); t.get(wf[k]); }
    }
    for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
        float xv[RMS_MAXV][8], gv[RMS_MAXV][8];
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < RMS_MAXV; ++k) {
            const int i = k * blockDim.x + threadIdx.x;
            if (i < nv) {
                Vec8<T> a, b;
                a.load(x + row * H + (size_t)i * 8);
                b.load(dy + row * H + (size_t)i * 8);
                a.get(xv[k]);
                b.get(gv[k]);
#pragma unroll
                for (int j = 0; j < 8; ++j) dot += gv[k][j] * wf[k][j] * xv[k][j];
            }
        }
        dot = block_reduce_sum(dot, sm);
        const float rs = rstd[row];
        const float c = dot * rs * rs * rs / (float)H;
#pragma unroll
        for (int k = 0; k < RMS_MAXV; ++k) {
            const int i = k * blockDim.x + threadIdx.x;
            if (i < nv) {
                float of[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    of[j] = rs * gv[k][j] * wf[k][j] - c * xv[k][j];
                    dwacc[k][j] += gv[k][j] * xv[k][j] * rs;
                }
                if (dresid) {
                    Vec8<T> r;
                    float rf[8];
                    r.load(dresid + row * H + (size_t)i * 8);
                    r.get(rf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) of[j] += rf[j];
                }
                Vec8<T> o;
                o.set(of);
                o.store(dx + row * H + (size_t)i * 8);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < RMS_MAXV; ++k) {
        const int i = k * blockDim.x + threadIdx.x;
        if (i < nv) {
            float* p = dw_partial + (size_t)blockIdx.x * H + (size_t)i * 8;
            reinterpret_cast<float4*>(p)[0] = make_float4(dwacc[k][0], dwacc[k][1], dwacc[k][2], dwacc[k][3]);
            reinterpret_cast<float4*>(p)[1] = make_float4(dwacc[k][4], dwacc[k][5], dwacc[k][6], dwacc[k][7]);
        }
    }
}

// out[c] = sum_p partial[p][c], written as T
template <typename T>
__global__ void colsum_kernel(const float* __restrict__ partial, int P, int H, T* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= H) return;
    float s = 0.f;
    for (int p = 0; p < P; ++p) s += partial[(size_t)p * H + c];
    out[c] = (T)s;
}
template <> __global__ void colsum_kernel<__nv_bfloat16>(const float* __restrict__ partial, int P, int H, __nv_bfloat16* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= H) return;
    float s = 0.f;
    for (int p = 0; p < P; ++p) s += partial[(size_t)p * H + c];
    out[c] = __float2bfloat16_rn(s);
}

// RMSNorm backward, one warp per row: the row's two reductions are warp shuffles (no block barrier per row), each lane
// owns up to MAXI 8-element vectors of the row, x / dy are read twice (the second pass hits L1).  A CTA's eight warps
// combine their dw sums through shared memory once, at the end.  H <= 256 * MAXI.
template <typename T, int MAXI>
__global__ void __launch_bounds__(256) rmsnorm_bwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                                                               const float* __restrict__ rstd, T* __restrict__ dx,
                                                               float* __restrict__ dw_partial, long long rows, int H,
                                                               const T* __restrict__ dresid) {
    __shared__ float sred[8][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nv = H / 8;
    float dwacc[MAXI][8];
#pragma unroll
    for (int k = 0; k < MAXI; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[k][j] = 0.f;
    for (long long row = (long long)blockIdx.x * 8 + warp; row < rows; row += (long long)gridDim.x * 8) {
        const T* xr = x + row * H;
        const T* gr = dy + row * H;
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < MAXI; ++k) {
            const int i = k * 32 + lane;
            if (i < nv) {
                Vec8<T> a, b, c;
                float xf[8], gf[8], wf[8];
                a.load(xr + (size_t)i * 8); b.load(gr + (size_t)i * 8); c.load(w + (size_t)i * 8);
                a.get(xf); b.get(gf); c.get(wf);
#pragma unroll
                for (int j = 0; j < 8; ++j) dot += gf[j] * wf[j] * xf[j];
            }
        }
        dot = warp_sum(dot);
        const float rs = rstd[row];
        const float cc = dot * rs * rs * rs / (float)H;
#pragma unroll
        for (int k = 0; k < MAXI; ++k) {
            const int i = k * 32 + lane;
            if (i < nv) {
                Vec8<T> a, b, c, o;
                float xf[8], gf[8], wf[8], of[8];
                a.load(xr + (size_t)i * 8); b.load(gr + (size_t)i * 8); c.load(w + (size_t)i * 8);
                a.get(xf); b.get(gf); c.get(wf);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    of[j] = rs * gf[j] * wf[j] - cc * xf[j];
                    dwacc[k][j] += gf[j] * xf[j] * rs;
                }
                if (dresid) {
                    Vec8<T> r;
                    float rf[8];
                    r.load(dresid + row * H + (size_t)i * 8);
                    r.get(rf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) of[j] += rf[j];
                }
                o.set(of);
                o.store(dx + row * H + (size_t)i * 8);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < MAXI; ++k) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sred[warp][lane * 8 + j] = dwacc[k][j];
        __syncthreads();
        {
            const int e = threadIdx.x;                     // element e of this item's 256
            const int i = k * 32 + (e >> 3);
            if (i < nv) {
                float t = 0.f;
#pragma unroll
                for (int ww = 0; ww < 8; ++ww) t += sred[ww][e];
                dw_partial[(size_t)blockIdx.x * H + (size_t)i * 8 + (e & 7)] = t;
            }
        }
        __syncthreads();
    }
}

// out[c] = sum_p partial[p][c]: 32 columns per CTA, eight row groups summed in parallel, then combined.
template <typename T>
__global__ void __launch_bounds__(256) colsum2_kernel(const float* __restrict__ partial, int P, int H, T* __restrict__ out) {
    __shared__ float sm[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < H)
        for (int p = ry; p < P; p += 8) s += partial[(size_t)p * H + c];
    sm[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < H) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) t += sm[r][cx];
        out[c] = (T)t;
    }
}

// ------------------------------------------------------------------------------------------ rotary embedding
// x: [B, T, heads, D] (contiguous), cos/sin: [T, D/2] fp32.  sign = +1 forward, -1 backward (the transpose).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ cs, const float* __restrict__ sn,
                            long long n_pairs, int Tlen, int heads, int D, int neox, float sign, int pos_offset) {
    const int half = D / 2;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_pairs; idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % half);
        const long long hv = idx / half;                       // (b*T + t)*heads + h
        const int t = (int)((hv / heads) % Tlen) + pos_offset;
        const float c = cs[(size_t)t * half + i], s = sn[(size_t)t * half + i] * sign;
        const size_t base = (size_t)hv * D;
        const size_t i0 = neox ? base + i : base + 2 * i, i1 = neox ? base + i + half : base + 2 * i + 1;
        const float a = (float)x[i0], b = (float)x[i1];
        y[i0] = (T)(a * c - b * s);
        y[i1] = (T)(b * c + a * s);
    }
}

// Fused split + rotary embedding of a packed projection: qkv [rows, (H + 2 Hk) D] (q heads, then k heads, then v heads;
// row = b * T + t) -> q [rows, H, D] and k [rows, Hk, D] rotated, v [rows, Hk, D] copied.  Backward (sign = -1) runs the
// other way: dq, dk, dv -> dqkv with the inverse rotation.  16 bytes per access; one pass over the data instead of two
// rotary launches and three strided copies.
template <typename T, bool BWD>
__global__ void qkv_rope_split_kernel(T* __restrict__ qkv, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                      const float* __restrict__ cs, const float* __restrict__ sn, long long rows, int Tlen, int H, int Hk,
                                      int D, int neox, int pos_offset) {
    const int half = D / 2, nh = H + Hk;
    const int per_head = neox ? D / 16 : D / 8;                 // rotation items per head: a lo/hi vector pair, or one vector of 4 pairs
    const long long n_rot = rows * nh * per_head, n_copy = rows * Hk * (D / 8);
    const int ld = (H + 2 * Hk) * D;
    const float sign = BWD ? -1.f : 1.f;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_rot + n_copy; idx += (long long)gridDim.x * blockDim.x) {
        if (idx < n_rot) {
            const int c = (int)(idx % per_head);
            const long long rh = idx / per_head;
            const int h = (int)(rh % nh);
            const long long row = rh / nh;
            const int t = (int)(row % Tlen) + pos_offset;
            T* packed = qkv + row * ld + (size_t)h * D;
            T* split = h < H ? q + (row * H + h) * D : k + (row * Hk + (h - H)) * D;
            T* src = BWD ? split : packed;
            T* dst = BWD ? packed : split;
            if (neox) {
                Vec8<T> lo, hi, olo, ohi;
                float a[8], b[8], oa[8], ob[8];
                lo.load(src + c * 8);
                hi.load(src + half + c * 8);
                lo.get(a);
                hi.get(b);
                const float4 c0 = reinterpret_cast<const float4*>(cs + (size_t)t * half + c * 8)[0], c1 = reinterpret_cast<const float4*>(cs + (size_t)t * half + c * 8)[1];
                const float4 s0 = reinterpret_cast<const float4*>(sn + (size_t)t * half + c * 8)[0], s1 = reinterpret_cast<const float4*>(sn + (size_t)t * half + c * 8)[1];
                const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    oa[j] = a[j] * cc[j] - b[j] * ss[j] * sign;
                    ob[j] = b[j] * cc[j] + a[j] * ss[j] * sign;
                }
                olo.set(oa);
                ohi.set(ob);
                olo.store(dst + c * 8);
                ohi.store(dst + half + c * 8);
            } else {
                Vec8<T> x, o;
                float a[8], oa[8];
                x.load(src + c * 8);
                x.get(a);
                const float4 c4 = *reinterpret_cast<const float4*>(cs + (size_t)t * half + c * 4);
                const float4 s4 = *reinterpret_cast<const float4*>(sn + (size_t)t * half + c * 4);
                const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    oa[2 * j] = a[2 * j] * cc[j] - a[2 * j + 1] * ss[j] * sign;
                    oa[2 * j + 1] = a[2 * j + 1] * cc[j] + a[2 * j] * ss[j] * sign;
                }
                o.set(oa);
                o.store(dst + c * 8);
            }
        } else {
            const long long i = idx - n_rot;
            const int c = (int)(i % (D / 8));
            const long long rh = i / (D / 8);
            const int h = (int)(rh % Hk);
            const long long row = rh / Hk;
            T* packed = qkv + row * ld + (size_t)(H + Hk + h) * D + c * 8;
            T* split = v + (row * Hk + h) * D + c * 8;
            Vec8<T> x;
            x.load(BWD ? split : packed);
            x.store(BWD ? packed : split);
        }
    }
}

// ------------------------------------------------------------------------------------------ gated activation
// gu: [rows, 2*I] with the gate in columns [0, I) and the up projection in [I, 2I); out: [rows, I].
template <typename T>
__global__ void gated_act_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int I, int gelu) {
    const int nv = I / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < rows * nv; v += (long long)gridDim.x * blockDim.x) {
        const long long r = v / nv;
        const int c = (int)(v % nv) * 8;
        Vec8<T> g, u, o;
        float gf[8], uf[8], of[8];
        g.load(gu + r * 2 * I + c);
        u.load(gu + r * 2 * I + I + c);
        g.get(gf);
        u.get(uf);
#pragma unroll
        for (int j = 0; j < 8; ++j) of[j] = (gelu ? gelu_tanh(gf[j]) : silu(gf[j])) * uf[j];
        o.set(of);
        o.store(out + r * I + c);
    }
}
template <typename T>
__global__ void gated_act_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout, T* __restrict__ dgu, long long rows, int I,
                                     int gelu) {
    const int nv = I / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < rows * nv; v += (long long)gridDim.x * blockDim.x) {
        const long long r = v / nv;
        const int c = (int)(v % nv) * 8;
        Vec8<T> g, u, d, og, ou;
        float gf[8], uf[8], df[8], a[8], b[8];
        g.load(gu + r * 2 * I + c);
        u.load(gu + r * 2 * I + I + c);
        d.load(dout + r * I + c);
        g.get(gf);
        u.get(uf);
        d.get(df);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float act, dact;
            if (gelu) {
                const float k = 0.7978845608028654f, x = gf[j];
                const float t = tanhf(k * (x + 0.044715f * x * x * x));
                act = 0.5f * x * (1.f + t);
                dact = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
            } else {
                const float sg = 1.f / (1.f + __expf(-gf[j]));
                act = gf[j] * sg;
                dact = sg * (1.f + gf[j] * (1.f - sg));
            }
            a[j] = df[j] * uf[j] * dact;
            b[j] = df[j] * act;
        }
        og.set(a);
        ou.set(b);
        og.store(dgu + r * 2 * I + c);
        ou.store(dgu + r * 2 * I + I + c);
    }
}

// ------------------------------------------------------------------------------------------ softmax + cross-entropy
// One CTA per row.  Pass 1: online max / sum-exp over the vocabulary.  loss = lse - logit[target].
// Pass 2 (if dlogits): dlogits = (softmax - onehot) * grad_scale, written in place or to a second buffer.
// Rows whose target equals ignore_index produce zero loss and zero gradient.
template <typename T>
__global__ void __launch_bounds__(1024) xent_fwd_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                                          float* __restrict__ loss, float* __restrict__ lse_out, T* __restrict__ dlogits,
                                                          int V, long long ld, float grad_scale, long long ignore_index) {
    __shared__ float sm[32];
    const size_t row = blockIdx.x;
    const T* lp = logits + row * ld;
    const long long tgt = target[row];
    const int nv = V / 8;                     // vector part; the tail (V % 8) is handled element-wise
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        Vec8<T> t;
        float f[8];
        t.load(lp + (size_t)i * 8);
        t.get(f);
        float lm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
        const float nm = fmaxf(m, lm);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
        s = s * __expf(m - nm) + acc;
        m = nm;
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
        const float f = (float)lp[i];
        const float nm = fmaxf(m, f);
        s = s * __expf(m - nm) + __expf(f - nm);
        m = nm;
    }
    const float M = block_reduce_max(m, sm);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - M);
    const float S = block_reduce_sum(s, sm);
    const float lse = M + logf(S);
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
    if (threadIdx.x == 0) {
        loss[row] = ignored ? 0.f : lse - (float)lp[tgt];
        if (lse_out) lse_out[row] = lse;
    }
    if (!dlogits) return;
    T* dp = dlogits + row * ld;
    const float gs = ignored ? 0.f : grad_scale;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        Vec8<T> t, o;
        float f[8];
        t.load(lp + (size_t)i * 8);
        t.get(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float p = __expf(f[j] - lse);
            if ((long long)i * 8 + j == tgt) p -= 1.f;
            f[j] = p * gs;
        }
        o.set(f);
        o.store(dp + (size_t)i * 8);
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
        float p = __expf((float)lp[i] - lse);
        if (i == tgt) p -= 1.f;
        dp[i] = (T)(p * gs);
    }
}

}  // namespace ptb

using namespace ptb;

static int rms_threads(int H) {
    int t = (H / 8 + RMS_MAXV - 1) / RMS_MAXV;
    t = (t + 31) / 32 * 32;
    return t < 32 ? 32 : t;
}

#define PTB_DISPATCH_T(bf16, ...)                         \
    if (bf16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
    else { using T = float; __VA_ARGS__; }

PTB_API int ptb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps,
                            const void* resid_in, void* resid_out, int bf16, cudaStream_t st) {
    if (H % 8 || rms_threads(H) > 1024) { ptb_set_error("rmsnorm: hidden size %d must be a multiple of 8 and at most %d", H, 8 * RMS_MAXV * 1024); return -1; }
    if (rows == 0) return 0;
    PTB_DISPATCH_T(bf16, rmsnorm_fwd_kernel<T><<<(unsigned)rows, rms_threads(H), 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, H, eps, (const T*)resid_in, (T*)resid_out));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Both backward entry points (caller-provided scratch, static scratch) launch the same two kernels.
template <typename T>
static void launch_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, float* dw_partial,
                               int n_ctas, long long rows, int H, const void* dresid, cudaStream_t st) {
    if (H <= 2048) {
        rmsnorm_bwd_warp_kernel<T, 8><<<n_ctas, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)dy, rstd, (T*)dx, dw_partial, rows, H, (const T*)dresid);
    } else if (H <= 4096) {
        rmsnorm_bwd_warp_kernel<T, 16><<<n_ctas, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)dy, rstd, (T*)dx, dw_partial, rows, H, (const T*)dresid);
    } else {
        rmsnorm_bwd_kernel<T><<<n_ctas, rms_threads(H), 0, st>>>((const T*)x, (const T*)w, (const T*)dy, rstd, (T*)dx, dw_partial, (int)rows, H, (const T*)dresid);
    }
    colsum2_kernel<T><<<(H + 31) / 32, 256, 0, st>>>(dw_partial, n_ctas, H, (T*)dw);
}

// dw_partial: [n_ctas, H] fp32 scratch.
PTB_API int ptb_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, float* dw_partial,
                            int n_ctas, long long rows, int H, const void* dresid, int bf16, cudaStream_t st) {
    if (H % 8 || rms_threads(H) > 1024) { ptb_set_error("rmsnorm: hidden size %d not supported", H); return -1; }
    if (rows == 0) return 0;
    PTB_DISPATCH_T(bf16, launch_rmsnorm_bwd<T>(x, w, dy, rstd, dx, dw, dw_partial, n_ctas, rows, H, dresid, st));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_rope(const void* x, void* y, const float* cos, const float* sin, long long B, int T_, int heads, int D, int neox,
                     int backward, int pos_offset, int bf16, cudaStream_t st) {
    const long long n_pairs = B * T_ * heads * (D / 2);
    if (n_pairs == 0) return 0;
    const int grid = (int)std::min<long long>((n_pairs + 255) / 256, 148LL * 16);
    PTB_DISPATCH_T(bf16, rope_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (T*)y, cos, sin, n_pairs, T_, heads, D, neox, backward ? -1.f : 1.f, pos_offset));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Forward: qkv -> (q, k rotated; v).  Backward (backward != 0): (dq, dk, dv) -> dqkv with the inverse rotation.
// rows = B * T; cos/sin fp32 [>= pos_offset + T, D/2]; D a multiple of 16.
PTB_API int ptb_qkv_rope_split(void* qkv, void* q, void* k, void* v, const float* cos, const float* sin, long long rows, int T_, int H, int Hk,
                               int D, int neox, int pos_offset, int backward, int bf16, cudaStream_t st) {
    if (D % 16) { ptb_set_error("qkv_rope_split: head size %d must be a multiple of 16", D); return -1; }
    if (rows == 0) return 0;
    const long long items = rows * (H + Hk) * (neox ? D / 16 : D / 8) + rows * Hk * (D / 8);
    const int grid = (int)std::min<long long>((items + 255) / 256, 148LL * 16);
    if (backward) {
        PTB_DISPATCH_T(bf16, qkv_rope_split_kernel<T, true><<<grid, 256, 0, st>>>((T*)qkv, (T*)q, (T*)k, (T*)v, cos, sin, rows, T_, H, Hk, D, neox, pos_offset));
    } else {
        PTB_DISPATCH_T(bf16, qkv_rope_split_kernel<T, false><<<grid, 256, 0, st>>>((T*)qkv, (T*)q, (T*)k, (T*)v, cos, sin, rows, T_, H, Hk, D, neox, pos_offset));
    }
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_gated_act_fwd(const void* gu, void* out, long long rows, int I, int gelu, int bf16, cudaStream_t st) {
    if (I % 8) { ptb_set_error("gated activation: width %d must be a multiple of 8", I); return -1; }
    if (rows == 0) return 0;
    const int grid = (int)std::min<long long>((rows * (I / 8) + 255) / 256, 148LL * 16);
    PTB_DISPATCH_T(bf16, gated_act_fwd_kernel<T><<<grid, 256, 0, st>>>((const T*)gu, (T*)out, rows, I, gelu));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_gated_act_bwd(const void* gu, const void* dout, void* dgu, long long rows, int I, int gelu, int bf16, cudaStream_t st) {
    if (I % 8) { ptb_set_error("gated activation: width %d must be a multiple of 8", I); return -1; }
    if (rows == 0) return 0;
    const int grid = (int)std::min<long long>((rows * (I / 8) + 255) / 256, 148LL * 16);
    PTB_DISPATCH_T(bf16, gated_act_bwd_kernel<T><<<grid, 256, 0, st>>>((const T*)gu, (const T*)dout, (T*)dgu, rows, I, gelu));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// logits [rows, ld] (V valid columns), target int64 [rows]; loss fp32 [rows]; dlogits may alias logits or be null.
PTB_API int ptb_xent(const void* logits, const long long* target, float* loss, float* lse, void* dlogits, long long rows, int V,
                     long long ld, float grad_scale, long long ignore_index, int bf16, cudaStream_t st) {
    if (rows == 0) return 0;
    if (ld % 8) { ptb_set_error("cross entropy: row stride %lld must be a multiple of 8 elements", ld); return -1; }
    const int threads = V >= 8192 ? 1024 : V >= 2048 ? 512 : V >= 512 ? 128 : 32;
    PTB_DISPATCH_T(bf16, xent_fwd_bwd_kernel<T><<<(unsigned)rows, threads, 0, st>>>((const T*)logits, target, loss, lse, (T*)dlogits, V, ld, grad_scale, ignore_index));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------------------------------ no-allocation variant
// RMSNorm backward with its scratch in the library image instead of a caller's buffer (see no_alloc.h).
// Host programs without an allocator of their own, and loops that must not touch the device allocator
// while they run, call this one; the partial sums land in `g_rms_static_scratch`, shared by every call
// on the device.
#include "no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_rms_static_scratch[PTB_RMS_STATIC_SCRATCH_FLOATS];

PTB_API int ptb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, int n_ctas,
                                   long long rows, int H, const void* dresid, int bf16, cudaStream_t st) {
    constexpr int MAX_DEV = 64;
    static float* scratch_of[MAX_DEV] = {nullptr};
    static std::mutex mu;
    if (H % 8 || H <= 0 || rms_threads(H) > 1024) { ptb_set_error("rmsnorm: hidden size %d not supported", H); return -1; }
    if (n_ctas <= 0) { ptb_set_error("rmsnorm_bwd_static: n_ctas must be positive"); return -1; }
    if ((long long)n_ctas * H > (long long)PTB_RMS_STATIC_SCRATCH_FLOATS) {
        ptb_set_error("rmsnorm_bwd_static: n_ctas * H = %lld exceeds the static scratch of %d floats; use fewer CTAs or ptb_rmsnorm_bwd",
                      (long long)n_ctas * H, (int)PTB_RMS_STATIC_SCRATCH_FLOATS);
        return -1;
    }
    if (rows == 0) return 0;
    int dev = 0;
    PTB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEV) { ptb_set_error("rmsnorm_bwd_static: device index %d out of range", dev); return -1; }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!scratch_of[dev]) {                       // once per device: where does this device keep the array?
            float* p = nullptr;
            PTB_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_rms_static_scratch));
            scratch_of[dev] = p;
        }
        scratch = scratch_of[dev];
    }
    PTB_DISPATCH_T(bf16, launch_rmsnorm_bwd<T>(x, w, dy, rstd, dx, dw, scratch, n_ctas, rows, H, dresid, st));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
