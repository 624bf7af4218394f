// Kernels of layer parts that are not attention and not a matrix product:
//   * token embedding + sinusoidal position vector + layer norm -> float32 residual stream
//   * gated residual sum + layer norm (weight, no bias)
//   * short causal convolution over time with a per-request state of the last inputs
//   * RMS norm of the two latents of a latent-attention mixer, the key/value latent written to
//     its cache slot
//   * the xIELU activation
// Everything a norm, a gate or a position computes is float32; inputs and outputs are float32 or
// bfloat16.  One CTA per token (row) unless stated otherwise.
#include "common.cuh"
#include "vec4.cuh"

namespace somi {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// Mean and inverse standard deviation of the H floats in `buf` (shared memory), two passes:
// the variance is the mean of the squared deviations from the mean.
__device__ __forceinline__ void mean_rstd(const float* buf, int H, float eps, float* scratch,
                                          float& mean, float& rstd) {
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += buf[i];
    mean = block_sum(s, scratch) / static_cast<float>(H);
    float v = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = buf[i] - mean;
        v = fmaf(d, d, v);
    }
    rstd = 1.0f / sqrtf(block_sum(v, scratch) / static_cast<float>(H) + eps);
}

// ------------------------------------------- embedding + sinusoid + layer norm
// x = table[ids[t]] + s(positions[t]);  s[2i] = sin(p * inv_freq[i]), s[2i+1] = cos(same angle)
// (inv_freq[i] = base^(-2i/H), made on the host);
// residual[t] = (x - mean) * rstd * weight.
template <typename T>
__global__ void embed_sinusoid_layernorm_kernel(const int* __restrict__ ids,
                                                const int* __restrict__ positions,
                                                const T* __restrict__ table,
                                                const float* __restrict__ inv_freq,
                                                const void* __restrict__ weight, int weight_dtype,
                                                float eps, float* __restrict__ out, int H) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + static_cast<size_t>(ids[t]) * H;
    const float p = static_cast<float>(positions[t]);
    for (int pair = threadIdx.x; 2 * pair < H; pair += blockDim.x) {
        const float angle = p * inv_freq[pair];        // float32, rounded once
        float sn, cs;
        sincosf(angle, &sn, &cs);
        row_buf[2 * pair] = to_float(row[2 * pair]) + sn;
        if (2 * pair + 1 < H) row_buf[2 * pair + 1] = to_float(row[2 * pair + 1]) + cs;
    }
    __syncthreads();
    float mean, rstd;
    mean_rstd(row_buf, H, eps, scratch, mean, rstd);
    float* o = out + static_cast<size_t>(t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = (row_buf[i] - mean) * rstd * load_as_float(weight, weight_dtype, i);
}

// ------------------------------------------------ gated residual + layer norm
// r = residual[row] + g * sum_s delta[s][row], g = sigmoid(gate[row]) (1 without a gate);
// if write_back: residual[row] = r;  out[b] = (r - mean) * rstd * weight  (rms = 1: r * rrms * weight),
// row = rows ? rows[b] : b.  delta: [splits] partial sums `split_stride` elements apart, added in order;
// the gate's logits may be partial sums of the same kind.  `extra`: float32 rows [N, H] that are
// added too, outside the gate (a second branch of the same layer).
template <typename TD, typename TG, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                     int splits, long long split_stride,
                                     const TG* __restrict__ gate, long long gate_stride,
                                     int gate_splits, long long gate_split_stride,
                                     const void* __restrict__ weight, int weight_dtype, float eps,
                                     TO* __restrict__ out, const int* __restrict__ rows, int H,
                                     int write_back, int rms, int vec4,
                                     const float* __restrict__ extra) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const size_t row = rows ? static_cast<size_t>(rows[b]) : static_cast<size_t>(b);
    float* r = residual + row * H;
    const float* x = extra ? extra + row * H : nullptr;
    const TD* d = delta ? delta + row * H : nullptr;
    const TG* g = gate ? gate + row * gate_stride : nullptr;
    TO* o = out + static_cast<size_t>(b) * H;
    if (vec4 && H <= static_cast<int>(blockDim.x) * 16) {
        // Up to four vectors of four columns a thread, every load of the row issued before the
        // first sum is needed; the row stays in registers between the passes.
        F4 v[4];
        const int step = blockDim.x * 4;
        const int i0 = threadIdx.x * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (i0 + k * step < H) v[k] = load4(r + i0 + k * step);
        if (d) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * step;
                if (i < H) {
                    F4 sum = load4(d + i);
                    for (int sp = 1; sp < splits; ++sp) {
                        const F4 t = load4(d + sp * split_stride + i);
#pragma unroll
                        for (int e = 0; e < 4; ++e) sum.v[e] += t.v[e];
                    }
                    if (g) {
                        F4 gg = load4(g + i);
                        for (int sp = 1; sp < gate_splits; ++sp) {
                            const F4 t = load4(g + sp * gate_split_stride + i);
#pragma unroll
                            for (int e = 0; e < 4; ++e) gg.v[e] += t.v[e];
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) sum.v[e] *= sigmoid_f(gg.v[e]);
                    }
                    if (x) {
                        const F4 t = load4(x + i);
#pragma unroll
                        for (int e = 0; e < 4; ++e) sum.v[e] += t.v[e];
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[k].v[e] += sum.v[e];
                    if (write_back) store4(r + i, v[k]);
                }
            }
        }
        float mean = 0.f;
        if (!rms) {
            float sm = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (i0 + k * step < H) sm += (v[k].v[0] + v[k].v[1]) + (v[k].v[2] + v[k].v[3]);
            mean = block_sum(sm, scratch) / static_cast<float>(H);
        }
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (i0 + k * step < H) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float dv = v[k].v[e] - mean;
                    ss = fmaf(dv, dv, ss);
                }
            }
        const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(H) + eps);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * step;
            if (i < H) {
                const F4 w = load4_any(weight, weight_dtype, i);
                F4 y;
#pragma unroll
                for (int e = 0; e < 4; ++e) y.v[e] = (v[k].v[e] - mean) * rstd * w.v[e];
                store4(o + i, y);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (d) {
            float sum = to_float(d[i]);
            for (int sp = 1; sp < splits; ++sp) sum += to_float(d[sp * split_stride + i]);
            if (g) {
                float gg = to_float(g[i]);
                for (int sp = 1; sp < gate_splits; ++sp) gg += to_float(g[sp * gate_split_stride + i]);
                sum *= sigmoid_f(gg);
            }
            if (x) sum += x[i];
            v += sum;
            if (write_back) r[i] = v;
        }
        row_buf[i] = v;
    }
    __syncthreads();
    float mean = 0.f, rstd;
    if (rms) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(row_buf[i], row_buf[i], ss);
        rstd = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(H) + eps);
    } else {
        mean_rstd(row_buf, H, eps, scratch, mean, rstd);
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_float<TO>((row_buf[i] - mean) * rstd * load_as_float(weight, weight_dtype, i));
}

// ------------------------------------------------- short causal convolution
// out[t] = h[t] + sum_{d=0}^{taps-1} w[taps-1-d, :] * h_(t-d) (w: [taps, H]), where h_(t-d) is the row d places
// back in the same request: a row of this step, or (before the step's first row) the request's
// state, which holds its last taps-1 inputs, oldest first, zero before the sequence's start.
// The state is only read here; `causal_taps_state_kernel` moves it on afterwards.
template <typename T>
__global__ void causal_taps_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                   const T* __restrict__ state, const int* __restrict__ cu_q,
                                   const int* __restrict__ token_request,
                                   const int* __restrict__ state_slot, T* __restrict__ out, int H,
                                   int taps, int vec4, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    // blockDim.y tokens a CTA: the look-ups that lead to a token's rows (request, first row,
    // slot) are a chain of dependent loads, and several chains run side by side
    const int t = blockIdx.x * blockDim.y + threadIdx.y;
    if (t >= n_tokens) return;
    const int req = token_request[t];
    const int local = t - cu_q[req];
    const T* st = state + static_cast<size_t>(state_slot[req]) * (taps - 1) * H;
    if (vec4) {
        for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < H; c += gridDim.y * blockDim.x * 4) {
            const F4 own = load4(h + static_cast<size_t>(t) * H + c);
            F4 acc = F4{{0.f, 0.f, 0.f, 0.f}};
            for (int d = taps - 1; d >= 0; --d) {      // oldest input first
                const F4 v = d == 0 ? own
                             : (local - d >= 0 ? load4(h + static_cast<size_t>(t - d) * H + c)
                                               : load4(st + static_cast<size_t>(taps - 1 + local - d) * H + c));
                const F4 ww = load4(w + static_cast<size_t>(taps - 1 - d) * H + c);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc.v[e] = fmaf(ww.v[e], v.v[e], acc.v[e]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) acc.v[e] += own.v[e];
            store4(out + static_cast<size_t>(t) * H + c, acc);
        }
        return;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
        const float own = to_float(h[static_cast<size_t>(t) * H + c]);
        float acc = 0.f;
        for (int d = taps - 1; d >= 0; --d) {          // oldest input first
            float v;
            if (d == 0) v = own;
            else if (local - d >= 0) v = to_float(h[static_cast<size_t>(t - d) * H + c]);
            else v = to_float(st[static_cast<size_t>(taps - 1 + local - d) * H + c]);
            acc = fmaf(w[static_cast<size_t>(taps - 1 - d) * H + c], v, acc);
        }
        out[static_cast<size_t>(t) * H + c] = from_float<T>(own + acc);
    }
}

// A step in which every request brings one token: output and new state in one kernel.  A thread
// owns four channels of one request: it reads the state's rows, then shifts them by one.
template <typename T>
__global__ void causal_taps_single_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                          T* __restrict__ state, const int* __restrict__ state_slot,
                                          T* __restrict__ out, int H, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    T* st = state + static_cast<size_t>(state_slot[t]) * (taps - 1) * H;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < H; c += gridDim.y * blockDim.x * 4) {
        const F4 own = load4(h + static_cast<size_t>(t) * H + c);
        const F4 w_own = load4(w + static_cast<size_t>(taps - 1) * H + c);
        F4 acc;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc.v[e] = w_own.v[e] * own.v[e];
        for (int s = 0; s < taps - 1; ++s) {               // state row s is the input taps-1-s back
            const F4 v = load4(st + static_cast<size_t>(s) * H + c);
            const F4 ww = load4(w + static_cast<size_t>(s) * H + c);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc.v[e] = fmaf(ww.v[e], v.v[e], acc.v[e]);
            if (s > 0) store4(st + static_cast<size_t>(s - 1) * H + c, v);
        }
        if (taps > 1) store4(st + static_cast<size_t>(taps - 2) * H + c, own);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc.v[e] += own.v[e];
        store4(out + static_cast<size_t>(t) * H + c, acc);
    }
}

// New state of request r: its last taps-1 inputs after this step's rows, oldest first.  A thread
// owns one channel of one request and reads what it needs of the old state before it writes.
constexpr int kMaxTaps = 32;
template <typename T>
__global__ void causal_taps_state_kernel(const T* __restrict__ h, T* __restrict__ state,
                                         const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slot, int H, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.x;
    const int first = cu_q[req], q = cu_q[req + 1] - first;
    const int keep = taps - 1;
    T* st = state + static_cast<size_t>(state_slot[req]) * keep * H;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
        T v[kMaxTaps];
        for (int s = 0; s < keep; ++s) {
            const int local = q - keep + s;        // row of this step, or (negative) of the old state
            v[s] = local >= 0 ? h[static_cast<size_t>(first + local) * H + c]
                              : st[static_cast<size_t>(keep + local) * H + c];
        }
        for (int s = 0; s < keep; ++s) st[static_cast<size_t>(s) * H + c] = v[s];
    }
}

// ------------------------------------------ RMS norm of latents + cache write
// x[t] = [a (na columns) | b (nb columns)], rows `stride` elements apart; x may be `splits` float32
// partial sums `split_stride` elements apart, added in order.  a_out[t] = rmsnorm(a) * wa;
// rmsnorm(b) * wb goes to cache + slot_map[t] * nb (and nowhere when nb == 0).  One warp per part,
// two tokens per CTA.
template <typename TI, typename T>
__global__ void latent_norm_store_kernel(const TI* __restrict__ x, long long stride, int splits,
                                         long long split_stride, int na, int nb,
                                         const void* __restrict__ wa, const void* __restrict__ wb,
                                         int weight_dtype, float eps, T* __restrict__ a_out,
                                         const int* __restrict__ slot_map, T* __restrict__ cache,
                                         int T_rows, int vec4) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 6) + (warp >> 1);      // two warps per token
    const int part = warp & 1;
    if (t >= T_rows || (part == 1 && nb == 0)) return;
    const TI* src = x + static_cast<size_t>(t) * stride + (part == 0 ? 0 : na);
    const int n = part == 0 ? na : nb;
    const void* w = part == 0 ? wa : wb;
    T* dst = part == 0 ? a_out + static_cast<size_t>(t) * na
                       : cache + static_cast<size_t>(slot_map[t]) * nb;
    float ss = 0.f;
    if (vec4) {
        for (int i = lane * 4; i < n; i += 128) {
            F4 v = load4(src + i);
            for (int sp = 1; sp < splits; ++sp) {
                const F4 u = load4(src + sp * split_stride + i);
#pragma unroll
                for (int e = 0; e < 4; ++e) v.v[e] += u.v[e];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v.v[e], v.v[e], ss);
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(n) + eps);
        for (int i = lane * 4; i < n; i += 128) {
            F4 v = load4(src + i);
            for (int sp = 1; sp < splits; ++sp) {
                const F4 u = load4(src + sp * split_stride + i);
#pragma unroll
                for (int e = 0; e < 4; ++e) v.v[e] += u.v[e];
            }
            const F4 ww = load4_any(w, weight_dtype, i);
#pragma unroll
            for (int e = 0; e < 4; ++e) v.v[e] = v.v[e] * inv * ww.v[e];
            store4(dst + i, v);
        }
        return;
    }
    for (int i = lane; i < n; i += 32) {
        float v = to_float(src[i]);
        for (int sp = 1; sp < splits; ++sp) v += to_float(src[sp * split_stride + i]);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(n) + eps);
    for (int i = lane; i < n; i += 32) {
        float v = to_float(src[i]);
        for (int sp = 1; sp < splits; ++sp) v += to_float(src[sp * split_stride + i]);
        dst[i] = from_float<T>(v * inv * load_as_float(w, weight_dtype, i));
    }
}

// The same for the few rows of a decode step: a CTA per (token, latent), a thread per four
// columns, so that every load of the row (and of its partial sums) is in flight at once.
template <typename TI, typename T>
__global__ void latent_norm_store_wide_kernel(const TI* __restrict__ x, long long stride, int splits,
                                              long long split_stride, int na, int nb,
                                              const void* __restrict__ wa,
                                              const void* __restrict__ wb, int weight_dtype,
                                              float eps, T* __restrict__ a_out,
                                              const int* __restrict__ slot_map,
                                              T* __restrict__ cache) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const TI* src = x + static_cast<size_t>(t) * stride + (part == 0 ? 0 : na);
    const int n = part == 0 ? na : nb;
    const void* w = part == 0 ? wa : wb;
    T* dst = part == 0 ? a_out + static_cast<size_t>(t) * na
                       : cache + static_cast<size_t>(slot_map[t]) * nb;
    const int i = threadIdx.x * 4;          // n <= 4 * blockDim.x, n a multiple of 4
    F4 v = F4{{0.f, 0.f, 0.f, 0.f}};
    if (i < n) {
        v = load4(src + i);
        for (int sp = 1; sp < splits; ++sp) {
            const F4 u = load4(src + sp * split_stride + i);
#pragma unroll
            for (int e = 0; e < 4; ++e) v.v[e] += u.v[e];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) ss = fmaf(v.v[e], v.v[e], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(n) + eps);
    if (i < n) {
        const F4 ww = load4_any(w, weight_dtype, i);
#pragma unroll
        for (int e = 0; e < 4; ++e) v.v[e] = v.v[e] * inv * ww.v[e];
        store4(dst + i, v);
    }
}

// ---------------------------------------------------------------- xIELU
// z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2; (p, q) = act[0..1].
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ x, long long stride, const void* __restrict__ act,
                             int act_dtype, T* __restrict__ out, int n, int vec4) {
    pdl_launch_dependents();
    const float ap = softplus_f(load_as_float(act, act_dtype, 0));        // [constant]
    const float aq = 0.5f + softplus_f(load_as_float(act, act_dtype, 1));  // [constant]
    pdl_wait();
    const T* src = x + static_cast<size_t>(blockIdx.x) * stride;
    T* dst = out + static_cast<size_t>(blockIdx.x) * n;
    if (vec4) {
        // eight columns a thread and step: two vectors in flight
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < n; i += gridDim.y * blockDim.x * 8) {
            F4 z[2];
            z[0] = load4(src + i);
            if (i + 4 < n) z[1] = load4(src + i + 4);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                if (i + 4 * k >= n) break;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = z[k].v[e];
                    // bfloat16 results carry 8 bits: the fast exponential is enough there
                    const float em1 = sizeof(T) == 2 ? __expf(v) - 1.0f : expm1f(v);
                    z[k].v[e] = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(aq, em1 - v, 0.5f * v);
                }
                store4(dst + i + 4 * k, z[k]);
            }
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        const float z = to_float(src[i]);
        const float y = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
        dst[i] = from_float<T>(y);
    }
}

inline int row_threads(int H) { return H >= 4096 ? 512 : (H >= 1024 ? 256 : 128); }

}  // namespace somi

using namespace somi;

SOMI_API int somi_embed_sinusoid_layernorm(const int* ids, const int* positions, const void* table,
                                           int dtype, const float* inv_freq, const void* weight, int weight_dtype,
                                           float eps, float* out, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t smem = static_cast<size_t>(H) * sizeof(float);
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
#define SOMI_LAUNCH_EMB(TT)                                                                      \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(embed_sinusoid_layernorm_kernel<TT>,                            \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        launch_pdl(embed_sinusoid_layernorm_kernel<TT>, dim3(T), dim3(row_threads(H)), smem,     \
                   stream, ids, positions, static_cast<const TT*>(table), inv_freq, weight,      \
                   weight_dtype, eps, out, H);                                                   \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_EMB(float);
    else SOMI_LAUNCH_EMB(__nv_bfloat16);
#undef SOMI_LAUNCH_EMB
    return launch_status();
}

SOMI_API int somi_add_layernorm(float* residual, const void* delta, int delta_dtype, int delta_splits,
                                long long delta_split_stride, const void* gate, int gate_dtype,
                                long long gate_stride, int gate_splits, long long gate_split_stride,
                                const void* weight, int weight_dtype, float eps,
                                void* out, int out_dtype, const int* rows, int n_out, int H,
                                int write_back, int rms, const float* extra, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (delta_splits < 1 || (delta_splits > 1 && delta_dtype != SOMI_F32)) return SOMI_ERR_UNSUPPORTED;
    if (gate && !delta) return SOMI_ERR_UNSUPPORTED;
    if (gate_splits < 1 || (gate_splits > 1 && gate_dtype != SOMI_F32)) return SOMI_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>(H) * sizeof(float);
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    if (!gate) gate_dtype = out_dtype;
    const int vec4 = (H & 3) == 0 && (gate_stride & 3) == 0 && (delta_split_stride & 3) == 0 &&
                     (gate_split_stride & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(gate) |
                       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(weight) |
                       reinterpret_cast<uintptr_t>(extra)) & 15) == 0;
    if (extra != nullptr && delta == nullptr) return SOMI_ERR_UNSUPPORTED;
    // few rows (a decode step waits for this kernel): a thread per four columns, the row read
    // in one pass; many rows: fewer threads per row, more rows per SM
    int threads = row_threads(H);
    if (vec4 && (n_out <= 32 || (delta_splits > 1 && n_out <= 256)))
        threads = min(1024, ((H / 4 + 31) / 32) * 32);
#define SOMI_LAUNCH_LN(TD, TG, TO)                                                               \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(add_layernorm_kernel<TD, TG, TO>,                               \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        launch_pdl(add_layernorm_kernel<TD, TG, TO>, dim3(n_out), dim3(threads), smem,           \
                   stream, residual, static_cast<const TD*>(delta), delta_splits,                \
                   delta_split_stride, static_cast<const TG*>(gate), gate_stride, gate_splits,   \
                   gate_split_stride, weight,                                                    \
                   weight_dtype, eps, static_cast<TO*>(out), rows, H, write_back, rms, vec4,     \
                   extra);                                                                       \
    } while (0)
    // the output is of the compute dtype; the delta and the gate are that or float32 partial sums
    if (out_dtype == SOMI_F32) {
        if (delta_dtype != SOMI_F32 || gate_dtype != SOMI_F32) return SOMI_ERR_UNSUPPORTED;
        SOMI_LAUNCH_LN(float, float, float);
    } else if (gate_dtype == SOMI_BF16) {
        if (delta_dtype == SOMI_F32) SOMI_LAUNCH_LN(float, __nv_bfloat16, __nv_bfloat16);
        else SOMI_LAUNCH_LN(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    } else {     // float32 logits: partial sums of a split-K product
        if (delta_dtype == SOMI_F32) SOMI_LAUNCH_LN(float, float, __nv_bfloat16);
        else SOMI_LAUNCH_LN(__nv_bfloat16, float, __nv_bfloat16);
    }
#undef SOMI_LAUNCH_LN
    return launch_status();
}

// ------------------------------------------------ stream + pending sums, beside a second stream
// out[t] = [residual[t] + sum_s delta[s][t] + extra[t] | tail[t]] in the compute dtype, 2 H wide:
// the input of a product that re-mixes the stream with another one (float32 sums, one rounding).
template <typename TD, typename TO>
__global__ void add_concat_kernel(const float* __restrict__ residual, const TD* __restrict__ delta,
                                  int splits, long long split_stride, const float* __restrict__ extra,
                                  const float* __restrict__ tail, TO* __restrict__ out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    const float* r = residual + row * H;
    const float* tl = tail + row * H;
    TO* o = out + row * 2 * H;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float v = r[i];
        if (delta != nullptr) {
            float sum = to_float(delta[row * H + i]);
            for (int sp = 1; sp < splits; ++sp) sum += to_float(delta[sp * split_stride + row * H + i]);
            if (extra != nullptr) sum += extra[row * H + i];
            v += sum;
        }
        o[i] = from_float<TO>(v);
        o[H + i] = from_float<TO>(tl[i]);
    }
}

SOMI_API int somi_add_concat(const float* residual, const void* delta, int delta_dtype, int splits,
                             long long split_stride, const float* extra, const float* tail, void* out,
                             int out_dtype, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || splits < 1 || (splits > 1 && delta_dtype != SOMI_F32) ||
        (extra != nullptr && delta == nullptr))
        return SOMI_ERR_UNSUPPORTED;
    const int threads = min(256, ((H + 31) / 32) * 32);
    if (!delta) delta_dtype = out_dtype;
#define SOMI_LAUNCH_AC(TD, TO)                                                                   \
    launch_pdl(add_concat_kernel<TD, TO>, dim3(T, T <= 256 ? (H + threads - 1) / threads : 1),   \
               dim3(threads), 0, stream, residual,                                               \
               static_cast<const TD*>(delta), splits, split_stride, extra, tail,                 \
               static_cast<TO*>(out), H)
    if (out_dtype == SOMI_F32) {
        if (delta_dtype != SOMI_F32) return SOMI_ERR_UNSUPPORTED;
        SOMI_LAUNCH_AC(float, float);
    } else if (delta_dtype == SOMI_F32) SOMI_LAUNCH_AC(float, __nv_bfloat16);
    else SOMI_LAUNCH_AC(__nv_bfloat16, __nv_bfloat16);
#undef SOMI_LAUNCH_AC
    return launch_status();
}

SOMI_API int somi_causal_taps_max() { return kMaxTaps; }

// h, out: [T, H]; w: float32 [taps, H]; state: [slots, taps - 1, H] of h's dtype.
SOMI_API int somi_causal_taps(const void* h, int dtype, const float* w, void* state, const int* cu_q,
                              const int* token_request, const int* state_slot, void* out, int T,
                              int R, int H, int taps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > kMaxTaps || R <= 0) return SOMI_ERR_UNSUPPORTED;
    const int vec4 = (H & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
    const int per_thread = vec4 ? 4 : 1;
    const int threads = min(256, ((H / per_thread + 31) / 32) * 32);
    const int ychunks = max(1, min(16, (H / per_thread + threads - 1) / threads));
    const int tb = min(256, ((H + 31) / 32) * 32);
    const int chunks = max(1, min(64, (H + tb - 1) / tb));
#define SOMI_LAUNCH_TAPS(TT)                                                                     \
    do {                                                                                         \
        if (T == R && vec4) {                                                                    \
            launch_pdl(causal_taps_single_kernel<TT>, dim3(T, ychunks), dim3(threads), 0, stream,\
                       static_cast<const TT*>(h), w, static_cast<TT*>(state), state_slot,        \
                       static_cast<TT*>(out), H, taps);                                          \
            break;                                                                               \
        }                                                                                        \
        launch_pdl(causal_taps_kernel<TT>, dim3((T + 3) / 4, max(1, min(4, H / 1024))),          \
                   dim3(64, 4), 0, stream,                                                       \
                   static_cast<const TT*>(h), w, static_cast<const TT*>(state), cu_q,            \
                   token_request, state_slot, static_cast<TT*>(out), H, taps, vec4, T);          \
        if (taps > 1)                                                                            \
            launch_pdl(causal_taps_state_kernel<TT>, dim3(R, chunks), dim3(tb), 0, stream,       \
                       static_cast<const TT*>(h), static_cast<TT*>(state), cu_q, state_slot, H,  \
                       taps);                                                                    \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_TAPS(float);
    else SOMI_LAUNCH_TAPS(__nv_bfloat16);
#undef SOMI_LAUNCH_TAPS
    return launch_status();
}

SOMI_API int somi_latent_norm_store(const void* x, int dtype, long long stride, int splits,
                                    long long split_stride, int na, int nb, const void* wa,
                                    const void* wb, int weight_dtype, float eps, void* a_out,
                                    int out_dtype, const int* slot_map, void* cache, int T,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (na <= 0 || nb < 0 || (nb > 0 && (!slot_map || !cache))) return SOMI_ERR_UNSUPPORTED;
    if (splits < 1 || (splits > 1 && dtype != SOMI_F32)) return SOMI_ERR_UNSUPPORTED;
    if (dtype != out_dtype && !(dtype == SOMI_F32 && out_dtype == SOMI_BF16)) return SOMI_ERR_UNSUPPORTED;
    const int vec4 = ((na | nb | static_cast<int>(stride & 3) | static_cast<int>(split_stride & 3)) & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a_out) |
                       reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(wa) |
                       reinterpret_cast<uintptr_t>(wb)) & 15) == 0;
#define SOMI_LAUNCH_LAT(TI, TT)                                                                  \
    launch_pdl(latent_norm_store_kernel<TI, TT>, dim3((T + 1) / 2), dim3(128), 0, stream,        \
               static_cast<const TI*>(x), stride, splits, split_stride, na, nb, wa, wb,          \
               weight_dtype, eps, static_cast<TT*>(a_out), slot_map, static_cast<TT*>(cache), T, \
               vec4)
    const int widest = max(na, nb);
    if (vec4 && T <= 64 && widest <= 4096) {
        const int threads = ((widest / 4 + 31) / 32) * 32;
#define SOMI_LAUNCH_LATW(TI, TT)                                                                 \
    launch_pdl(latent_norm_store_wide_kernel<TI, TT>, dim3(T, nb > 0 ? 2 : 1), dim3(threads), 0, \
               stream, static_cast<const TI*>(x), stride, splits, split_stride, na, nb, wa, wb,  \
               weight_dtype, eps, static_cast<TT*>(a_out), slot_map, static_cast<TT*>(cache))
        if (out_dtype == SOMI_F32) SOMI_LAUNCH_LATW(float, float);
        else if (dtype == SOMI_F32) SOMI_LAUNCH_LATW(float, __nv_bfloat16);
        else SOMI_LAUNCH_LATW(__nv_bfloat16, __nv_bfloat16);
#undef SOMI_LAUNCH_LATW
        return launch_status();
    }
    if (out_dtype == SOMI_F32) SOMI_LAUNCH_LAT(float, float);
    else if (dtype == SOMI_F32) SOMI_LAUNCH_LAT(float, __nv_bfloat16);
    else SOMI_LAUNCH_LAT(__nv_bfloat16, __nv_bfloat16);
#undef SOMI_LAUNCH_LAT
    return launch_status();
}

SOMI_API int somi_xielu(const void* x, int dtype, long long stride, const void* act, int act_dtype,
                        void* out, int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const int vec4 = ((n | static_cast<int>(stride & 3)) & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int threads = 256;
    const int per_cta = threads * (vec4 ? 8 : 1);
    // few rows: the row's columns over several CTAs; many rows: a CTA walks a part of the row
    const int ychunks = T >= 512 ? max(1, min(8, n / (2 * per_cta))) : max(1, min(64, (n + per_cta - 1) / per_cta));
    if (dtype == SOMI_F32)
        launch_pdl(xielu_kernel<float>, dim3(T, ychunks), dim3(threads), 0, stream,
                   static_cast<const float*>(x), stride, act, act_dtype, static_cast<float*>(out), n,
                   vec4);
    else
        launch_pdl(xielu_kernel<__nv_bfloat16>, dim3(T, ychunks), dim3(threads), 0, stream,
                   static_cast<const __nv_bfloat16*>(x), stride, act, act_dtype,
                   static_cast<__nv_bfloat16*>(out), n, vec4);
    return launch_status();
}
