// Mixture of experts.  Which experts a token uses is a table row of `top` expert numbers: the row of
// its token id in a table of the model (ids given), or its own row of a table that a router filled
// for this step (ids null).
//
//   router:   softmax over the router's logits, a correction added for the choice only, the best
//             `keep` of `count` groups of neighbouring experts by their best member, the `top` best
//             members of those; the weights are the softmax values of the chosen.
//   route:    for every (token, k) pair ("entry" t * top + k) the expert table[row, k]; entries are
//             grouped by expert (a counting sort in one CTA) and the groups are cut into row tiles.
//             Experts numbered E and above have no matrices ("identity experts": their output is
//             their input); their entries are placed behind the others and get no tile.
//   grouped product: one CTA per (row tile of an expert's entries, tile of output columns),
//             C = A W_e^T with float32 FMAs, every output summed over K in ascending order, so an
//             entry's result does not depend on the tile it fell into or on the rest of the step.
//             Epilogues: the experts' gated activation over row-interleaved gate/up weights, or
//             float32 rows scattered back to the entries' places.
//   matrix-vector: a step of few entries needs no grouping: every entry streams the rows of its
//             own expert (bfloat16, 16-byte loads, two rows a warp), with the same two epilogues.
//   gather / activation: what stands around the library's grouped product in prompt-sized
//             bfloat16 steps: the rows in the grouped order, and the experts' gated activation.
//   combine:  out[t] = weight * sum_k y[row of entry t * top + k] (+ the shared expert's rows), float32;
//             or with a weight per entry, an identity expert's entry adding weight * x[t].
//
// A product over all rows with one weight matrix (a shared expert) is the same kernel with one
// group.  Everything is decided on the device: the launches depend on the step's layout only.
#include "common.cuh"
#include "vec4.cuh"

namespace somi {

constexpr int kMoeBM = 32;       // entries per row tile
constexpr int kMoeBN = 64;       // output columns per CTA
constexpr int kMoeBK = 32;
constexpr int kMoeThreads = 256;

// offsets: int32 [E + 1] first sorted position of every expert; sorted: int32 [n_entries] entry
// ids grouped by expert; tile_expert / tile_row0: int32 [max_tiles], n_tiles: int32 [1];
// place: int32 [n_entries] the sorted position of every entry (the inverse of `sorted`).
__global__ void moe_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, int T,
                                 int top, int E, int E_all, int* __restrict__ offsets, int* __restrict__ sorted,
                                 int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                 int* __restrict__ n_tiles, int max_tiles, int* __restrict__ place) {
    extern __shared__ int sm[];          // counts [E_all], cursor [E_all]
    int* counts = sm;
    int* cursor = sm + E_all;
    pdl_launch_dependents();
    pdl_wait();
    const int n = T * top;
    for (int e = threadIdx.x; e < E_all; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = table[static_cast<size_t>(ids != nullptr ? ids[i / top] : i / top) * top + i % top];
        if (e >= 0 && e < E_all) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E_all; ++e) {
            if (e <= E) offsets[e] = at;
            cursor[e] = at;
            for (int r = 0; e < E && r < counts[e] && tiles < max_tiles; r += kMoeBM) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = at + r;
                ++tiles;
            }
            at += counts[e];
        }
        if (E_all == E) offsets[E] = at;
        *n_tiles = tiles;
    }
    __syncthreads();
    // one atomic per entry places it in its expert's group; the order inside a group changes no
    // result (each entry's row is computed by itself)
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = table[static_cast<size_t>(ids != nullptr ? ids[i / top] : i / top) * top + i % top];
        if (e >= 0 && e < E_all) {
            const int pos = atomicAdd(&cursor[e], 1);
            sorted[pos] = i;
            place[i] = pos;
        }
    }
}

// out[p, :] = a[sorted[p] / top, :]: the rows of the step's tokens in the grouped order.
template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ a, long long a_stride,
                                       const int* __restrict__ sorted, int top, int K,
                                       T* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.x;
    const T* src = a + static_cast<size_t>(sorted[p] / top) * a_stride;
    T* dst = out + static_cast<size_t>(p) * K;
    if ((K & 7) == 0 && sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
        return;
    }
    for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
}

// The activation of an expert that has no gate: 0 gelu (erf), 1 gelu (tanh), 2 silu, 3 squared relu.
__device__ __forceinline__ float unary_act(float z, int kind) {
    switch (kind) {
        case 0: return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
        case 1: return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
        case 2: return z / (1.0f + expf(-z));
        default: { const float r = fmaxf(z, 0.f); return r * r; }
    }
}

template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    if (sizeof(T) == 2 && (n & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
            uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + i);
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                h[e] = __floats2bfloat162_rn(unary_act(__low2float(h[e]), kind), unary_act(__high2float(h[e]), kind));
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + i) = raw;
        }
        return;
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = from_float<T>(unary_act(to_float(x[i]), kind));
}

// The experts' activation over a product whose columns alternate gate_j, up_j:
// out[r, j] = g * sigmoid(alpha * g) * (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit)
// (limit = infinity, alpha = 1, shift = 0: silu(gate) * up).
template <typename T>
__global__ void clamped_gate_up_kernel(const T* __restrict__ gu, T* __restrict__ out, int ff,
                                       long long n, float limit, float alpha, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    if (sizeof(T) == 2 && (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        // four outputs a thread: eight inputs in one 16-byte load
        const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(gu);
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
        for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
            const uint4 raw = *reinterpret_cast<const uint4*>(in + 2 * i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float g = fminf(__low2float(h[e]), limit);
                const float u = fminf(fmaxf(__high2float(h[e]), -limit), limit);
                y[e] = g / (1.0f + expf(-alpha * g)) * (u + shift);
            }
            const __nv_bfloat162 y01 = __floats2bfloat162_rn(y[0], y[1]), y23 = __floats2bfloat162_rn(y[2], y[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&y01);
            packed.y = *reinterpret_cast<const uint32_t*>(&y23);
            *reinterpret_cast<uint2*>(o + i) = packed;
        }
        return;
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float g = fminf(to_float(gu[2 * i]), limit);
        const float u = fminf(fmaxf(to_float(gu[2 * i + 1]), -limit), limit);
        out[i] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

// A step of few tokens: every (token, k) entry streams the rows of its own expert.
// grid (row blocks, entries); a warp computes two weight rows at a time (a gate row and its up
// row, or two output rows), lanes stride over K with 16-byte loads; x of the entry sits in shared
// memory as float32.  MODE 1: the gated activation, out [entries, N / 2] bfloat16;
// MODE 0: out [entries, N] float32; MODE 2: an activation without a gate (`act`), out [entries, N]
// bfloat16.
constexpr int kGemvWarps = 8;
constexpr int kGemvRowsPerCta = 64;
template <int MODE>
__global__ void __launch_bounds__(kGemvWarps * 32)
moe_gemv_kernel(const __nv_bfloat16* __restrict__ A, long long a_stride, int a_div,
                const __nv_bfloat16* __restrict__ W, const int* __restrict__ ids,
                const int* __restrict__ table, int top, int E, void* __restrict__ out, int N, int K,
                float limit, float alpha, float shift, int act) {
    extern __shared__ float xs[];                          // [K]
    pdl_launch_dependents();
    pdl_wait();
    const int entry = blockIdx.y;
    const int expert = table[static_cast<size_t>(ids != nullptr ? ids[entry / top] : entry / top) * top + entry % top];
    if (expert < 0 || expert >= E) return;
    const __nv_bfloat16* x = A + static_cast<size_t>(entry / a_div) * a_stride;
    for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = __bfloat162float(x[i]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __nv_bfloat16* Wm = W + static_cast<size_t>(expert) * N * K;
    const int row_end = min(N, (static_cast<int>(blockIdx.x) + 1) * kGemvRowsPerCta);
    for (int row = blockIdx.x * kGemvRowsPerCta + warp * 2; row < row_end; row += kGemvWarps * 2) {
        const __nv_bfloat16* w0 = Wm + static_cast<size_t>(row) * K;
        const __nv_bfloat16* w1 = w0 + K;
        const bool two = row + 1 < N;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 u0 = *reinterpret_cast<const uint4*>(w0 + k);
            const uint4 u1 = two ? *reinterpret_cast<const uint4*>(w1 + k) : make_uint4(0, 0, 0, 0);
            const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x0 = xs[k + 2 * e], x1 = xs[k + 2 * e + 1];
                a0 = fmaf(__low2float(h0[e]), x0, a0);
                a0 = fmaf(__high2float(h0[e]), x1, a0);
                a1 = fmaf(__low2float(h1[e]), x0, a1);
                a1 = fmaf(__high2float(h1[e]), x1, a1);
            }
        }
        a0 = warp_sum(a0);
        a1 = warp_sum(a1);
        if (lane == 0) {
            if (MODE == 1) {
                const float g = fminf(a0, limit);
                const float u = fminf(fmaxf(a1, -limit), limit);
                static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(entry) * (N / 2) + row / 2] =
                    __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + shift));
            } else if (MODE == 2) {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(entry) * N;
                o[row] = __float2bfloat16_rn(unary_act(a0, act));
                if (two) o[row + 1] = __float2bfloat16_rn(unary_act(a1, act));
            } else {
                float* o = static_cast<float*>(out) + static_cast<size_t>(entry) * N;
                o[row] = a0;
                if (two) o[row + 1] = a1;
            }
        }
    }
}

// MODE 0: out (TO) rows at `scatter` positions (or the sorted position itself), N columns.
// MODE 1: W's rows alternate gate_j, up_j; g = min(gate, limit), u = clamp(up, -limit, limit);
//         out[pos, j] = g * sigmoid(alpha * g) * (u + shift), N / 2 columns.
// MODE 2: out[pos, c] = act(product), N columns (an expert without a gate).
template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(kMoeThreads)
grouped_gemm_kernel(const T* __restrict__ A, long long a_stride, const int* __restrict__ gather,
                    int gather_div, const T* __restrict__ W, const int* __restrict__ offsets,
                    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    const int* __restrict__ n_tiles, int n_rows_single, TO* __restrict__ out,
                    long long out_stride, const int* __restrict__ scatter, int N, int K, float limit,
                    float alpha, float shift, int act) {
    __shared__ float As[kMoeBK][kMoeBM + 1];
    __shared__ float Ws[kMoeBK][kMoeBN + 1];
    __shared__ int rows_s[kMoeBM];
    pdl_launch_dependents();
    pdl_wait();
    int expert = 0, row0, row_end;
    if (tile_expert != nullptr) {
        if (static_cast<int>(blockIdx.x) >= *n_tiles) return;
        expert = tile_expert[blockIdx.x];
        row0 = tile_row0[blockIdx.x];
        row_end = offsets[expert + 1];
    } else {                                   // one group: all rows, weight matrix 0
        row0 = blockIdx.x * kMoeBM;
        row_end = n_rows_single;
        if (row0 >= row_end) return;
    }
    const int rows = min(kMoeBM, row_end - row0);
    const int col0 = blockIdx.y * kMoeBN;
    const int tid = threadIdx.x;
    if (tid < kMoeBM) {
        int src = -1;
        if (tid < rows) {
            src = row0 + tid;
            if (gather != nullptr) src = gather[src] / gather_div;
        }
        rows_s[tid] = src;
    }
    __syncthreads();
    const T* Wm = W + static_cast<size_t>(expert) * N * K;
    const int ty = tid / 16, tx = tid % 16;     // rows ty*2.., columns tx*4..
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kMoeBK) {
        for (int idx = tid; idx < kMoeBM * kMoeBK; idx += kMoeThreads) {
            const int m = idx / kMoeBK, kk = idx % kMoeBK;
            const int src = rows_s[m];
            As[kk][m] = (src >= 0 && k0 + kk < K)
                            ? to_float(A[static_cast<size_t>(src) * a_stride + k0 + kk]) : 0.f;
        }
        for (int idx = tid; idx < kMoeBN * kMoeBK; idx += kMoeThreads) {
            const int nn = idx / kMoeBK, kk = idx % kMoeBK;
            Ws[kk][nn] = (col0 + nn < N && k0 + kk < K)
                             ? to_float(Wm[static_cast<size_t>(col0 + nn) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kMoeBK; ++kk) {
            const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float w = Ws[kk][tx * 4 + j];
                acc[0][j] = fmaf(a0, w, acc[0][j]);
                acc[1][j] = fmaf(a1, w, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = ty * 2 + i;
        if (m >= rows) continue;
        const int pos = row0 + m;
        if (MODE == 0) {
            const size_t dst = static_cast<size_t>(scatter != nullptr ? scatter[pos] : pos) * out_stride;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = col0 + tx * 4 + j;
                if (c < N) out[dst + c] = from_float<TO>(acc[i][j]);
            }
        } else if (MODE == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = col0 + tx * 4 + j;
                if (c < N) out[static_cast<size_t>(pos) * out_stride + c] = from_float<TO>(unary_act(acc[i][j], act));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int c = col0 + tx * 4 + j;       // even: a gate row; c + 1 its up row
                if (c + 1 < N) {
                    const float g = fminf(acc[i][j], limit);
                    const float u = fminf(fmaxf(acc[i][j + 1], -limit), limit);
                    const float y = g / (1.0f + expf(-alpha * g)) * (u + shift);
                    out[static_cast<size_t>(pos) * out_stride + c / 2] = from_float<TO>(y);
                }
            }
        }
    }
}

// out[t, c] = weight * sum_k y[row(t * top + k), c] (+ extra[t, c]); float32.  row(e) = place[e]
// where the rows of y are in the grouped order, else e.
template <typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place,
                                   const float* __restrict__ extra, float weight, int top, int H,
                                   long long n, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    if ((H & 3) == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(extra) |
                          reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
            const long long t = i / H;
            const int c = static_cast<int>(i - t * H);
            F4 s = F4{{0.f, 0.f, 0.f, 0.f}};
            for (int k = 0; k < top; ++k) {
                const long long e = t * top + k;
                const F4 v = load4(y + (place != nullptr ? place[e] : e) * H + c);
#pragma unroll
                for (int q = 0; q < 4; ++q) s.v[q] += v.v[q];
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) s.v[q] *= weight;
            if (extra != nullptr) {
                const F4 x = load4(extra + i);
#pragma unroll
                for (int q = 0; q < 4; ++q) s.v[q] += x.v[q];
            }
            store4(out + i, s);
        }
        return;
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / H;
        const int c = static_cast<int>(i - t * H);
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const long long e = t * top + k;
            s += to_float(y[(place != nullptr ? place[e] : e) * H + c]);
        }
        s *= weight;
        if (extra != nullptr) s += extra[i];
        out[i] = s;
    }
}


// ------------------------------------------------------------------- router
// One warp per token.  s = softmax(logits[t, 0..n)) (float32); choice = s + correction (null: s);
// the n outputs form `count` equal groups of neighbours, a group's score is its largest choice, and
// only members of the `keep` best groups can be chosen (count <= 1: all can); the `top` largest
// choices among those are written to chosen[t, 0..top) in falling order, their s to weight[t, ..].
// Equal values go to the lower index.  With `over_chosen` the choice is made on the logits
// themselves (no correction, no groups) and the weights are the softmax over the chosen logits only.
__global__ void moe_router_select_kernel(const float* __restrict__ logits, long long l_stride,
                                         const float* __restrict__ correction, int n, int count,
                                         int keep, int top, int* __restrict__ chosen,
                                         float* __restrict__ weight, int T, int over_chosen) {
    extern __shared__ float rs[];            // per warp: s [n], choice [n], group score [count]
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    const int groups = count > 1 ? count : 1;
    float* sv = rs + static_cast<size_t>(warp) * (2 * n + groups);
    float* cv = sv + n;
    float* gv = cv + n;
    const float* z = logits + static_cast<size_t>(t) * l_stride;
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, z[i]);
    m = warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float e = expf(z[i] - m);
        sv[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < n; i += 32) {
        const float p = sv[i] / sum;
        sv[i] = p;
        cv[i] = over_chosen ? z[i] : (correction != nullptr ? p + correction[i] : p);
    }
    __syncwarp();
    if (count > 1 && keep < count) {
        const int size = n / count;
        for (int g = lane; g < count; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < size; ++i) best = fmaxf(best, cv[g * size + i]);
            gv[g] = best;
        }
        __syncwarp();
        // the (count - keep) worst groups leave: the best `keep` stay, marked by +infinity
        for (int round = 0; round < keep; ++round) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < count; g += 32) {
                const float v = gv[g];
                if (v != INFINITY && (v > best || (v == best && g < arg))) { best = v; arg = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (lane == 0 && arg != 0x7fffffff) gv[arg] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < n; i += 32)
            if (gv[i / size] != INFINITY) cv[i] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float v = cv[i];
            if (!isnan(v) && (v > best || (v == best && i < arg))) { best = v; arg = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;
        if (lane == 0) {
            chosen[static_cast<size_t>(t) * top + k] = arg;
            weight[static_cast<size_t>(t) * top + k] = sv[arg];
            cv[arg] = NAN;                    // taken: not chosen again
        }
        __syncwarp();
    }
    if (over_chosen && lane == 0) {           // the first chosen has the largest logit
        int* c = chosen + static_cast<size_t>(t) * top;
        float* w = weight + static_cast<size_t>(t) * top;
        const float zmax = z[c[0]];
        float den = 0.f;
        for (int k = 0; k < top; ++k) { w[k] = expf(z[c[k]] - zmax); den += w[k]; }
        for (int k = 0; k < top; ++k) w[k] /= den;
    }
}

// out[t, c] = sum_k weight[t, k] * (table[t, k] < E ? y[row(t * top + k), c] : x[t, c]); float32.
// row(e) = place[e] where the rows of y are in the grouped order, else e.  The sum runs over k in
// ascending order.
// A CTA per token (its entries of table, weight and place are read once by every warp); a thread
// four neighbouring columns where the rows allow it (`vec`), else one.
template <typename TY, typename TX>
__global__ void moe_combine_weighted_kernel(const TY* __restrict__ y, const int* __restrict__ place,
                                            const int* __restrict__ table,
                                            const float* __restrict__ weight, const TX* __restrict__ x,
                                            int E, int top, int H, int T, int vec, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        const long long e0 = static_cast<long long>(t) * top;
        const TX* xr = x + static_cast<size_t>(t) * H;
        float* o = out + static_cast<size_t>(t) * H;
        if (vec) {
            for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
                F4 s{{0.f, 0.f, 0.f, 0.f}};
                for (int k = 0; k < top; ++k) {
                    const int expert = table[e0 + k];
                    const float w = weight[e0 + k];
                    const F4 v = (expert >= 0 && expert < E)
                        ? load4(y + static_cast<size_t>(place != nullptr ? place[e0 + k] : e0 + k) * H + c)
                        : load4(xr + c);
#pragma unroll
                    for (int j = 0; j < 4; ++j) s.v[j] = fmaf(w, v.v[j], s.v[j]);
                }
                store4(o + c, s);
            }
        } else {
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                float s = 0.f;
                for (int k = 0; k < top; ++k) {
                    const int expert = table[e0 + k];
                    const float v = (expert >= 0 && expert < E)
                        ? to_float(y[static_cast<size_t>(place != nullptr ? place[e0 + k] : e0 + k) * H + c])
                        : to_float(xr[c]);
                    s = fmaf(weight[e0 + k], v, s);
                }
                o[c] = s;
            }
        }
    }
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_moe_row_tile() { return kMoeBM; }

// work: int32 [(E + 1) + n_entries + 2 * max_tiles + 1 + n_entries]: offsets, sorted, tile_expert,
// tile_row0, n_tiles, place
// Table entries in [E, E_all) are experts without matrices: placed behind the others, no tiles.
SOMI_API int somi_moe_route(const int* ids, const int* table, int T, int top, int E, int E_all,
                            int* work, int max_tiles, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (top <= 0 || E <= 0 || E_all < E || E_all > 4096) return SOMI_ERR_UNSUPPORTED;
    int* offsets = work;
    int* sorted = offsets + E + 1;
    int* tile_expert = sorted + static_cast<size_t>(T) * top;
    int* tile_row0 = tile_expert + max_tiles;
    int* n_tiles = tile_row0 + max_tiles;
    int* place = n_tiles + 1;
    launch_pdl(moe_route_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * E_all, stream, ids, table, T,
               top, E, E_all, offsets, sorted, tile_expert, tile_row0, n_tiles, max_tiles, place);
    return launch_status();
}

SOMI_API int somi_moe_gather_rows(const void* a, int dtype, long long a_stride, const int* work, int E,
                                  int n_entries, int top, int K, void* out, cudaStream_t stream) {
    if (n_entries <= 0) return 0;
    const int* sorted = work + E + 1;
    const int threads = min(256, max(32, ((K / 8 + 31) / 32) * 32));
    if (dtype == SOMI_F32)
        launch_pdl(moe_gather_rows_kernel<float>, dim3(n_entries), dim3(threads), 0, stream,
                   static_cast<const float*>(a), a_stride, sorted, top, K, static_cast<float*>(out));
    else
        launch_pdl(moe_gather_rows_kernel<__nv_bfloat16>, dim3(n_entries), dim3(threads), 0, stream,
                   static_cast<const __nv_bfloat16*>(a), a_stride, sorted, top, K,
                   static_cast<__nv_bfloat16*>(out));
    return launch_status();
}

SOMI_API int somi_clamped_gate_up(const void* gu, void* out, int dtype, long long rows, int ff,
                                  float limit, float alpha, float shift, cudaStream_t stream) {
    const long long n = rows * ff;
    if (n <= 0) return 0;
    const int blocks = static_cast<int>(((n + 255) / 256) < 148LL * 16 ? ((n + 255) / 256) : 148LL * 16);
    if (dtype == SOMI_F32)
        launch_pdl(clamped_gate_up_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const float*>(gu), static_cast<float*>(out), ff, n, limit, alpha, shift);
    else
        launch_pdl(clamped_gate_up_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), ff, n,
                   limit, alpha, shift);
    return launch_status();
}

SOMI_API int somi_unary_act(const void* x, void* out, int dtype, long long n, int kind,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 3) return SOMI_ERR_UNSUPPORTED;
    const int blocks = static_cast<int>(((n + 255) / 256) < 148LL * 16 ? ((n + 255) / 256) : 148LL * 16);
    if (dtype == SOMI_F32)
        launch_pdl(unary_act_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const float*>(x), static_cast<float*>(out), n, kind);
    else
        launch_pdl(unary_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n, kind);
    return launch_status();
}

// bfloat16, K a multiple of 8: mode 1 the gated activation (out bfloat16 [entries, N / 2]), mode 0
// float32 rows [entries, N].  Row e of A is a[e / a_div].
SOMI_API int somi_moe_gemv(const void* A, long long a_stride, int a_div, const void* W, const int* ids,
                           const int* table, int top, int E, int n_entries, void* out, int N, int K,
                           int mode, float limit, float alpha, float shift, int act, cudaStream_t stream) {
    if (n_entries <= 0) return 0;
    if (K <= 0 || (K & 7) || N <= 0 || (mode == 1 && (N & 1)) || K > 40 * 1024 ||
        (reinterpret_cast<uintptr_t>(W) & 15))
        return SOMI_ERR_UNSUPPORTED;
    dim3 grid((N + kGemvRowsPerCta - 1) / kGemvRowsPerCta, n_entries);
    const size_t smem = sizeof(float) * K;
    if (mode == 1) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(moe_gemv_kernel<1>, grid, dim3(kGemvWarps * 32), smem, stream,
                   static_cast<const __nv_bfloat16*>(A), a_stride, a_div,
                   static_cast<const __nv_bfloat16*>(W), ids, table, top, E, out, N, K, limit, alpha, shift, act);
    } else if (mode == 2) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(moe_gemv_kernel<2>, grid, dim3(kGemvWarps * 32), smem, stream,
                   static_cast<const __nv_bfloat16*>(A), a_stride, a_div,
                   static_cast<const __nv_bfloat16*>(W), ids, table, top, E, out, N, K, limit, alpha, shift, act);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_gemv_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(moe_gemv_kernel<0>, grid, dim3(kGemvWarps * 32), smem, stream,
                   static_cast<const __nv_bfloat16*>(A), a_stride, a_div,
                   static_cast<const __nv_bfloat16*>(W), ids, table, top, E, out, N, K, limit, alpha, shift, act);
    }
    return launch_status();
}

// mode 0: out[scatter ? scatter[pos] : pos] = A W^T rows (out_dtype 0: float32, 1: as A);
// mode 1: gated activation over interleaved gate/up rows (out as A).  `work` as somi_moe_route
// left it, or null for one group of `n_rows` rows (the weight is then one matrix).
SOMI_API int somi_grouped_gemm(const void* A, int dtype, long long a_stride, int gather_div,
                               int use_gather, const void* W, const int* work, int E, int n_entries,
                               int max_tiles, int n_rows, void* out, int out_f32,
                               long long out_stride, int use_scatter, int N, int K, int mode,
                               float limit, float alpha, float shift, int act, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return SOMI_ERR_UNSUPPORTED;
    const int* offsets = nullptr; const int* sorted = nullptr; const int* tile_expert = nullptr;
    const int* tile_row0 = nullptr; const int* n_tiles = nullptr;
    int tiles;
    if (work != nullptr) {
        offsets = work;
        sorted = offsets + E + 1;
        tile_expert = sorted + n_entries;
        tile_row0 = tile_expert + max_tiles;
        n_tiles = tile_row0 + max_tiles;
        tiles = max_tiles;
    } else {
        tiles = (n_rows + kMoeBM - 1) / kMoeBM;
    }
    if (tiles <= 0) return 0;
    if (mode == 1 && (N & 1)) return SOMI_ERR_UNSUPPORTED;
    dim3 grid(tiles, (N + kMoeBN - 1) / kMoeBN);
    const int* gather = use_gather ? sorted : nullptr;
    const int* scatter = use_scatter ? sorted : nullptr;
#define SOMI_LAUNCH_GG(TT, TO, MODE)                                                             \
    launch_pdl(grouped_gemm_kernel<TT, TO, MODE>, grid, dim3(kMoeThreads), 0, stream,            \
               static_cast<const TT*>(A), a_stride, gather, gather_div, static_cast<const TT*>(W), \
               offsets, tile_expert, tile_row0, n_tiles, n_rows, static_cast<TO*>(out), out_stride, \
               scatter, N, K, limit, alpha, shift, act)
    if (dtype == SOMI_F32) {
        if (mode == 1) SOMI_LAUNCH_GG(float, float, 1);
        else if (mode == 2) SOMI_LAUNCH_GG(float, float, 2);
        else SOMI_LAUNCH_GG(float, float, 0);
    } else {
        if (mode == 1) SOMI_LAUNCH_GG(__nv_bfloat16, __nv_bfloat16, 1);
        else if (mode == 2) SOMI_LAUNCH_GG(__nv_bfloat16, __nv_bfloat16, 2);
        else if (out_f32) SOMI_LAUNCH_GG(__nv_bfloat16, float, 0);
        else SOMI_LAUNCH_GG(__nv_bfloat16, __nv_bfloat16, 0);
    }
#undef SOMI_LAUNCH_GG
    return launch_status();
}

SOMI_API int somi_moe_combine(const void* y, int y_dtype, const int* place, const float* extra,
                              float weight, int top, int T, int H, float* out, cudaStream_t stream) {
    const long long n = static_cast<long long>(T) * H;
    if (n <= 0) return 0;
    const int blocks = static_cast<int>(((n + 255) / 256) < 148LL * 16 ? ((n + 255) / 256) : 148LL * 16);
    if (y_dtype == SOMI_F32)
        launch_pdl(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const float*>(y), place, extra, weight, top, H, n, out);
    else
        launch_pdl(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const __nv_bfloat16*>(y), place, extra, weight, top, H, n, out);
    return launch_status();
}

// logits: float32 [T, l_stride] (n columns read); chosen int32 [T, top], weight float32 [T, top].
SOMI_API int somi_moe_router_select(const float* logits, long long l_stride, const float* correction,
                                    int T, int n, int count, int keep, int top, int* chosen,
                                    float* weight, int over_chosen, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n <= 0 || n > 4096 || top <= 0 || top > n || (count > 1 && (n % count || keep <= 0 || keep > count)))
        return SOMI_ERR_UNSUPPORTED;
    if (count > 1 && keep < count && top > keep * (n / count)) return SOMI_ERR_UNSUPPORTED;
    const int warps = 4;
    const size_t smem = sizeof(float) * warps * (2 * n + (count > 1 ? count : 1));
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_router_select_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream,
               logits, l_stride, correction, n, count, keep, top, chosen, weight, T, over_chosen);
    return launch_status();
}

SOMI_API int somi_moe_combine_weighted(const void* y, int y_dtype, const int* place, const int* table,
                                       const float* weight, const void* x, int x_dtype, int E, int top,
                                       int T, int H, float* out, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    const int vec = (H % 4 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x) |
                                     reinterpret_cast<uintptr_t>(out)) & 15) == 0) ? 1 : 0;
    const int threads = min(256, max(32, ((H / (vec ? 4 : 1) + 31) / 32) * 32));
    const int blocks = min(T, 148 * 32);
#define SOMI_LAUNCH_CW(TY, TX)                                                                    \
    launch_pdl(moe_combine_weighted_kernel<TY, TX>, dim3(blocks), dim3(threads), 0, stream,       \
               static_cast<const TY*>(y), place, table, weight, static_cast<const TX*>(x), E, top, H, T, vec, out)
    if (y_dtype == SOMI_F32 && x_dtype == SOMI_F32) SOMI_LAUNCH_CW(float, float);
    else if (y_dtype == SOMI_F32) SOMI_LAUNCH_CW(float, __nv_bfloat16);
    else if (x_dtype == SOMI_F32) SOMI_LAUNCH_CW(__nv_bfloat16, float);
    else SOMI_LAUNCH_CW(__nv_bfloat16, __nv_bfloat16);
#undef SOMI_LAUNCH_CW
    return launch_status();
}
