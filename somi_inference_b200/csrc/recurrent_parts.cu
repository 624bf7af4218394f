// Kernels of layers whose branches run side by side and of mixers that carry a matrix state:
//   * residual += mult * (scale_a * a + scale_b * b), then one or two RMS norms of the same row
//     (a layer whose mixer and feed-forward both read the stream they both add to)
//   * RMS norm of every query and key head with a weight, rotation of the halves of a head's
//     first `rot` entries, cache write (keys and values of different widths)
//   * the recurrence of a matrix state per head, S <- decay * S + k u^T, o = S^T q, with
//     u = v (a decayed sum of outer products) or u = beta (v - S^T k) (the gated delta rule),
//     the decay a constant per head or a number per key channel and token
//   * RMS norm in equal parts of a row, times a weight, times the sigmoid of a gate
//   * half the sum of two rows, each RMS-normed with a weight of its own
//   * the square of relu
// Norms, angles, gates, decays, step sizes and the state are float32; inputs and outputs are float32
// or bfloat16.
#include "common.cuh"
#include "vec4.cuh"

namespace somi {

__device__ __forceinline__ float sigmoid32(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus32(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu32(float z) { return z / (1.0f + expf(-z)); }

// ------------------------------------- scaled sum of two branches + one or two RMS norms
// d_a = sum_s a[s][row] (partial sums `a_stride` apart, added in order), d_b likewise;
// r = residual[row] + mult * (scale_a .* d_a + scale_b .* d_b) + extra[row]   (an absent branch
// or absent extra rows add nothing);
// if write_back: residual[row] = r;  out1[i] = r / sqrt(mean(r^2) + eps) * w1, out2 likewise with
// w2 (either may be absent); row = rows ? rows[i] : i.  The row lives in shared memory.
__global__ void add_scaled_rmsnorm_kernel(float* __restrict__ residual, const void* __restrict__ a,
                                          int a_dtype, int a_splits, long long a_stride,
                                          const void* __restrict__ scale_a, const void* __restrict__ b,
                                          int b_dtype, int b_splits, long long b_stride,
                                          const void* __restrict__ scale_b, int scale_dtype, float mult,
                                          const float* __restrict__ extra,
                                          const void* __restrict__ w1, const void* __restrict__ w2,
                                          int w_dtype, float eps, void* __restrict__ out1,
                                          void* __restrict__ out2, int out_dtype,
                                          const int* __restrict__ rows, int H, int write_back, int vec4) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int i_out = blockIdx.x;
    const int row = rows ? rows[i_out] : i_out;
    float* res = residual + static_cast<size_t>(row) * H;
    const size_t base = static_cast<size_t>(row) * H;
    float ss = 0.f;
    if (vec4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            F4 r = load4(res + i);
            F4 t = F4{{0.f, 0.f, 0.f, 0.f}};
            if (a != nullptr) {
                F4 d = load4_any(a, a_dtype, base + i);
                for (int s = 1; s < a_splits; ++s) {
                    const F4 e = load4_any(a, a_dtype, static_cast<size_t>(s) * a_stride + base + i);
#pragma unroll
                    for (int c = 0; c < 4; ++c) d.v[c] += e.v[c];
                }
                if (scale_a != nullptr) {
                    const F4 sc = load4_any(scale_a, scale_dtype, i);
#pragma unroll
                    for (int c = 0; c < 4; ++c) d.v[c] *= sc.v[c];
                }
                t = d;
            }
            if (b != nullptr) {
                F4 d = load4_any(b, b_dtype, base + i);
                for (int s = 1; s < b_splits; ++s) {
                    const F4 e = load4_any(b, b_dtype, static_cast<size_t>(s) * b_stride + base + i);
#pragma unroll
                    for (int c = 0; c < 4; ++c) d.v[c] += e.v[c];
                }
                if (scale_b != nullptr) {
                    const F4 sc = load4_any(scale_b, scale_dtype, i);
#pragma unroll
                    for (int c = 0; c < 4; ++c) d.v[c] *= sc.v[c];
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) t.v[c] += d.v[c];
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) r.v[c] = fmaf(mult, t.v[c], r.v[c]);
            if (extra != nullptr) {
                const F4 x = load4(extra + base + i);
#pragma unroll
                for (int c = 0; c < 4; ++c) r.v[c] += x.v[c];
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) ss = fmaf(r.v[c], r.v[c], ss);
            store4(row_buf + i, r);
            if (write_back && (a != nullptr || b != nullptr || extra != nullptr)) store4(res + i, r);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float t = 0.f;
            if (a != nullptr) {
                float d = load_as_float(a, a_dtype, base + i);
                for (int s = 1; s < a_splits; ++s)
                    d += load_as_float(a, a_dtype, static_cast<size_t>(s) * a_stride + base + i);
                if (scale_a != nullptr) d *= load_as_float(scale_a, scale_dtype, i);
                t = d;
            }
            if (b != nullptr) {
                float d = load_as_float(b, b_dtype, base + i);
                for (int s = 1; s < b_splits; ++s)
                    d += load_as_float(b, b_dtype, static_cast<size_t>(s) * b_stride + base + i);
                if (scale_b != nullptr) d *= load_as_float(scale_b, scale_dtype, i);
                t += d;
            }
            float r = fmaf(mult, t, res[i]);
            if (extra != nullptr) r += extra[base + i];
            row_buf[i] = r;
            if (write_back && (a != nullptr || b != nullptr || extra != nullptr)) res[i] = r;
            ss = fmaf(r, r, ss);
        }
    }
    if (out1 == nullptr && out2 == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
    const size_t obase = static_cast<size_t>(i_out) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row_buf[i] * inv;
        if (out1 != nullptr) {
            const float y = v * load_as_float(w1, w_dtype, i);
            if (out_dtype == SOMI_F32) static_cast<float*>(out1)[obase + i] = y;
            else static_cast<__nv_bfloat16*>(out1)[obase + i] = __float2bfloat16_rn(y);
        }
        if (out2 != nullptr) {
            const float y = v * load_as_float(w2, w_dtype, i);
            if (out_dtype == SOMI_F32) static_cast<float*>(out2)[obase + i] = y;
            else static_cast<__nv_bfloat16*>(out2)[obase + i] = __float2bfloat16_rn(y);
        }
    }
}

// --------------------------- per-head RMS norm + rotation of halves + cache write
// A row of `qkv` holds nq query heads and nkv key heads of `hd` elements and nkv value heads of
// `vd` elements.  Every query and key head is divided by its root mean square over hd (eps inside
// the root) and multiplied by `q_w` / `k_w` (hd elements, shared by the heads; null: no norm);
// then entry i < rot/2 and entry i + rot/2 of the token at position p turn by p * inv_freq[i]
// (the angle is formed and reduced in float64, its sine and cosine are float32 and are both
// multiplied by `magnitude`, 1 for a plain rotation); entries from `rot` on pass.  Queries are written back in place; keys and values go to their cache slots.
// One warp per head; the normed head passes through shared memory so that a lane finds its partner.
template <typename T>
__global__ void headnorm_rotary_store_kernel(T* __restrict__ qkv, long long stride,
                                             const int* __restrict__ positions,
                                             const double* __restrict__ inv_freq, int nq, int nkv,
                                             int hd, int vd, int rot, const void* __restrict__ q_w,
                                             const void* __restrict__ k_w, int w_dtype, float eps,
                                             float magnitude,
                                             const int* __restrict__ slot_map, T* __restrict__ kcache,
                                             T* __restrict__ vcache, int page_size) {
    extern __shared__ float heads_s[];                 // [warps][hd]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    T* row = qkv + static_cast<size_t>(t) * stride;
    const double pos = static_cast<double>(positions[t]);
    const int slot = slot_map != nullptr ? slot_map[t] : -1;
    const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    float* mine = heads_s + warp * hd;
    const int half = rot >> 1;
    for (int head = blockIdx.y * nwarps + warp; head < nq + nkv; head += nwarps * gridDim.y) {
        T* x = row + static_cast<size_t>(head) * hd;
        const void* w = head < nq ? q_w : k_w;
        float ss = 0.f;
        for (int e = lane; e < hd; e += 32) {
            const float v = to_float(x[e]);
            mine[e] = v;
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (w != nullptr) {
            const float r = 1.0f / sqrtf(ss / static_cast<float>(hd) + eps);
            for (int e = lane; e < hd; e += 32) mine[e] = mine[e] * r * load_as_float(w, w_dtype, e);
        }
        __syncwarp();
        T* dst = nullptr;
        if (head < nq) dst = x;
        else if (slot >= 0) dst = kcache + ((page * nkv + (head - nq)) * page_size + off) * hd;
        if (dst != nullptr) {
            for (int e = lane; e < hd; e += 32) {
                float v = mine[e];
                if (e < rot) {
                    const int i = e < half ? e : e - half;
                    double angle = pos * inv_freq[i];
                    angle -= 6.283185307179586476925286766559 * rint(angle * 0.15915494309189533576888376337251);
                    float sn, cs;
                    sincosf(static_cast<float>(angle), &sn, &cs);
                    sn *= magnitude;
                    cs *= magnitude;
                    v = e < half ? fmaf(v, cs, -(mine[e + half] * sn)) : fmaf(v, cs, mine[e - half] * sn);
                }
                dst[e] = from_float<T>(v);
            }
        }
        __syncwarp();
    }
    if (slot >= 0 && blockIdx.y == 0) {
        const T* vrow = row + static_cast<size_t>(nq + nkv) * hd;
        for (int g = 0; g < nkv; ++g) {
            T* dst = vcache + ((page * nkv + g) * page_size + off) * vd;
            for (int e = threadIdx.x; e < vd; e += blockDim.x) dst[e] = vrow[static_cast<size_t>(g) * vd + e];
        }
    }
}

// ------------------------------------------------------- matrix-state recurrence
// Per request r and head h a state S [dk, dv] float32 in the request's slot (stored column by
// column, [dv][dk]); per token, in order:
//     S <- g .* S         g: decay[h] (a constant), or per key channel i
//                         g_i = exp(-exp(a_log[h]) * softplus(a[t, h dk + i] + dt_bias[h dk + i]))
//     u = v                                   (DELTA false)
//     u = sigmoid(b[t, h]) * (v - S^T k)      (DELTA true)
//     S <- S + k u^T;   y[t, h, :] = S^T q.
// q and k of head h are head h / (heads / qk_heads) of their tensors.  With `act_silu` q and k
// (bit 0) and v (bit 1) pass SiLU as they are read; with `unit` q and k are divided by
// sqrt(sum of squares + unit_eps); q is multiplied by q_scale either way.  v and beta are read by their
// own dtype code; with `decay_ready` a holds the decays g themselves.
// A CTA owns kRecCols columns of S for one (request, head) and walks through the request's rows
// of this step, B rows at a time (16, or 4 when no request has more rows than that).  Four warps
// hold the state, four columns each, every lane a few rows of all four (RecShape below); the sums
// over rows are taken in a fixed order (ascending in a lane, then the exchanges of rec_reduce4),
// so y does not depend on how the rows were cut into steps.  Four more warps stage the next block
// meanwhile: they read q, k, the decay logits, v and beta of its rows, apply the activations, the
// unit norms and the decay's exponentials (a warp per row) and leave float32 values in the other
// of two shared buffers.
constexpr int kRecLanes = 8;                             // key widths are padded to 8 R, R a power of two
constexpr int kRecWarps = 4;
constexpr int kRecLoaders = 4;
constexpr int kRecColsPerWarp = 4;
constexpr int kRecCols = kRecWarps * kRecColsPerWarp;
constexpr int kRecBlockLong = 16;                        // rows staged at a time in a long step
constexpr int kRecBlockShort = 4;                        // and in a step of few rows per request
constexpr int kRecThreads = (kRecWarps + kRecLoaders) * 32;

// floats of one staged block of B rows: q, k, g [B][DP], v [B][kRecCols], beta [B]
__host__ __device__ constexpr int rec_buffer_floats(int B, int DP) {
    return B * (3 * DP + kRecCols + 1);
}

// A state warp holds kRecColsPerWarp columns.  With DP = 8 R the padded key width, a lane holds
// RL = V J rows of each of them: J runs of V neighbours, entry (j, e) being row 32 V j + V lane + e
// (V = 4 from a width of 128 on, else DP / 32), so that the warp reads 32 V neighbouring floats of a
// staged row, or of a column of the state, with one access each, and the row's q, k and g are read
// once for all of the warp's columns.
template <int R>
struct RecShape {
    static constexpr int DP = R * kRecLanes;
    static constexpr int V = DP >= 128 ? 4 : DP / 32;
    static constexpr int J = DP / (32 * V);
    static constexpr int RL = V * J;
    static_assert(DP >= 32 && DP % 32 == 0, "a staged row is at least one float per lane");
};

// p: a staged row + V lane
template <int R>
__device__ __forceinline__ void rec_load_rows(const float* p, float (&out)[RecShape<R>::RL]) {
    constexpr int V = RecShape<R>::V;
#pragma unroll
    for (int j = 0; j < RecShape<R>::J; ++j) {
        if (V == 4) {
            const float4 x = *reinterpret_cast<const float4*>(p + j * 32 * V);
            out[4 * j] = x.x; out[4 * j + 1] = x.y; out[4 * j + 2] = x.z; out[4 * j + 3] = x.w;
        } else if (V == 2) {
            const float2 x = *reinterpret_cast<const float2*>(p + j * 32 * V);
            out[2 * j] = x.x; out[2 * j + 1] = x.y;
        } else {
            out[j] = p[j * 32];
        }
    }
}

// The rows of one column of a state (col: the column's dk floats) that `lane` holds, read into or
// written from s.  `runs`: dk is a multiple of V and the column starts on a 16-byte boundary, so
// a run of V rows is one access.
template <int R, bool STORE>
__device__ __forceinline__ void rec_state_rows(float* col, float (&s)[RecShape<R>::RL], int lane, int dk,
                                               bool live, bool runs) {
    constexpr int V = RecShape<R>::V;
#pragma unroll
    for (int j = 0; j < RecShape<R>::J; ++j) {
        const int row = 32 * V * j + V * lane;
        if (runs && V > 1) {
            const bool in = live && row < dk;
            if (V == 4) {
                float4* p = reinterpret_cast<float4*>(col + row);
                if (STORE) {
                    if (in) *p = make_float4(s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3]);
                } else {
                    const float4 x = in ? *p : make_float4(0.f, 0.f, 0.f, 0.f);
                    s[4 * j] = x.x; s[4 * j + 1] = x.y; s[4 * j + 2] = x.z; s[4 * j + 3] = x.w;
                }
            } else {
                float2* p = reinterpret_cast<float2*>(col + row);
                if (STORE) {
                    if (in) *p = make_float2(s[2 * j], s[2 * j + 1]);
                } else {
                    const float2 x = in ? *p : make_float2(0.f, 0.f);
                    s[2 * j] = x.x; s[2 * j + 1] = x.y;
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const bool in = live && row + e < dk;
                if (STORE) { if (in) col[row + e] = s[V * j + e]; }
                else s[V * j + e] = in ? col[row + e] : 0.f;
            }
        }
    }
}

// Four sums over the warp in six exchanges: lanes with bit 4 clear take columns 0 and 1 from
// their partner 16 away and give 2 and 3, then bit 3 halves the pair, then three butterfly steps.
// Every lane returns the warp's sum of d[2 * (lane bit 4) + (lane bit 3)]; the order of the
// additions is fixed.
__device__ __forceinline__ float rec_reduce4(const float (&d)[4], int lane) {
    const bool hi = (lane & 16) != 0, mid = (lane & 8) != 0;
    float a0 = hi ? d[2] : d[0], a1 = hi ? d[3] : d[1];
    a0 += __shfl_xor_sync(0xffffffffu, hi ? d[0] : d[2], 16);
    a1 += __shfl_xor_sync(0xffffffffu, hi ? d[1] : d[3], 16);
    float b = mid ? a1 : a0;
    b += __shfl_xor_sync(0xffffffffu, mid ? a0 : a1, 8);
    b += __shfl_xor_sync(0xffffffffu, b, 4);
    b += __shfl_xor_sync(0xffffffffu, b, 2);
    b += __shfl_xor_sync(0xffffffffu, b, 1);
    return b;
}

// The reverse: every lane holds the value of column 2 * (bit 4) + (bit 3); all get all four.
__device__ __forceinline__ void rec_gather4(float mine, int lane, float (&u)[4]) {
    const bool hi = (lane & 16) != 0, mid = (lane & 8) != 0;
    const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
    const float p0 = mid ? other : mine, p1 = mid ? mine : other;      // columns 2 hi, 2 hi + 1
    const float x0 = __shfl_xor_sync(0xffffffffu, p0, 16), x1 = __shfl_xor_sync(0xffffffffu, p1, 16);
    u[0] = hi ? x0 : p0; u[1] = hi ? x1 : p1; u[2] = hi ? p0 : x0; u[3] = hi ? p1 : x1;
}

template <typename T, int R, bool DELTA, int B>
__global__ void __launch_bounds__(kRecThreads, R > 16 ? 1 : (B == kRecBlockShort ? 4 : 2))
matrix_state_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const void* __restrict__ v,
                         int vb_dtype, long long q_stride, long long k_stride, long long v_stride,
                         int act_silu, int unit, float unit_eps, float q_scale,
                         const void* __restrict__ beta, long long beta_stride,
                         const float* __restrict__ a, long long a_stride, int decay_ready,
                         const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                         const float* __restrict__ decay, float* __restrict__ state,
                         const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                         float* __restrict__ y, int heads, int qk_heads, int dk, int dv) {
    constexpr int DP = R * kRecLanes;                    // padded key width
    constexpr int PL = (DP + 31) / 32;                   // key channels a staging lane holds
    constexpr int V = RecShape<R>::V, RL = RecShape<R>::RL;
    constexpr int kRowsPerLoader = B / kRecLoaders;
    constexpr int kValueLoads = (B * kRecCols + kRecLoaders * 32 - 1) / (kRecLoaders * 32);
    static_assert(B % kRecLoaders == 0, "a loader warp stages whole rows");
    static_assert(kRecColsPerWarp == 4, "the sums over the warp are taken four at a time");
    extern __shared__ __align__(16) float rec_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int qkh = h / (heads / qk_heads);
    const bool channel_decay = a != nullptr;
    const float head_decay = channel_decay ? 1.f : decay[h];
    const int first = cu_q[r], last = cu_q[r + 1];
    const int blocks = (last - first + B - 1) / B;
    const bool loader = warp >= kRecWarps;

    // ---- loaders: stage block `blk` into buffer `blk & 1`
    const float rate = channel_decay ? expf(a_log[h]) : 0.f;
    float bias[PL];
#pragma unroll
    for (int j = 0; j < PL; ++j) {
        const int i = lane + 32 * j;
        bias[j] = (loader && channel_decay && i < dk) ? dt_bias[static_cast<size_t>(h) * dk + i] : 0.f;
    }
    auto stage = [&](int blk) {
        float* buf = rec_smem + (blk & 1) * rec_buffer_floats(B, DP);
        float* q_s = buf;
        float* k_s = buf + B * DP;
        float* g_s = buf + 2 * B * DP;
        float* v_s = buf + 3 * B * DP;
        float* b_s = v_s + B * kRecCols;
        const int t0 = first + blk * B;
        const int n_tok = min(B, last - t0);
        const int lw = warp - kRecWarps, ltid = tid - kRecWarps * 32;
        // every load of the block's rows is issued before the first value is used
        float vv[kValueLoads];
#pragma unroll
        for (int j = 0; j < kValueLoads; ++j) {
            const int idx = ltid + kRecLoaders * 32 * j;
            const int tok = idx / kRecCols, cc = blockIdx.z * kRecCols + idx % kRecCols;
            vv[j] = (tok < n_tok && cc < dv)
                ? load_as_float(v, vb_dtype, static_cast<size_t>(t0 + tok) * v_stride + static_cast<size_t>(h) * dv + cc) : 0.f;
        }
        float bb = 0.f;
        if (DELTA && ltid < n_tok)
            bb = load_as_float(beta, vb_dtype, static_cast<size_t>(t0 + ltid) * beta_stride + h);
        float qv[kRowsPerLoader][PL], kv[kRowsPerLoader][PL], av[kRowsPerLoader][PL];
#pragma unroll
        for (int m = 0; m < kRowsPerLoader; ++m) {
            const int tok = lw + kRecLoaders * m;
            const size_t t = static_cast<size_t>(t0 + tok);
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                const int i = lane + 32 * j;
                const bool in = tok < n_tok && i < dk;
                qv[m][j] = in ? to_float(q[t * q_stride + static_cast<size_t>(qkh) * dk + i]) : 0.f;
                kv[m][j] = in ? to_float(k[t * k_stride + static_cast<size_t>(qkh) * dk + i]) : 0.f;
                av[m][j] = (in && channel_decay) ? a[t * a_stride + static_cast<size_t>(h) * dk + i] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < kValueLoads; ++j)
            if (ltid + kRecLoaders * 32 * j < B * kRecCols)
                v_s[ltid + kRecLoaders * 32 * j] = (act_silu & 2) ? silu32(vv[j]) : vv[j];
        if (DELTA && ltid < n_tok) b_s[ltid] = sigmoid32(bb);
#pragma unroll
        for (int m = 0; m < kRowsPerLoader; ++m) {
            const int tok = lw + kRecLoaders * m;
            if (tok >= n_tok) break;                       // uniform in the warp
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                if (act_silu & 1) { qv[m][j] = silu32(qv[m][j]); kv[m][j] = silu32(kv[m][j]); }
                sq = fmaf(qv[m][j], qv[m][j], sq);
                sk = fmaf(kv[m][j], kv[m][j], sk);
            }
            float rq = q_scale, rk = 1.f;
            if (unit) {                                    // the sum over the head in lane order
                sq = warp_sum(sq);
                sk = warp_sum(sk);
                rq = q_scale / sqrtf(sq + unit_eps);
                rk = 1.0f / sqrtf(sk + unit_eps);
            }
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                const int i = lane + 32 * j;
                if (i < DP) {
                    q_s[tok * DP + i] = qv[m][j] * rq;
                    k_s[tok * DP + i] = unit ? kv[m][j] * rk : kv[m][j];
                    g_s[tok * DP + i] = (channel_decay && i < dk)
                        ? (decay_ready ? av[m][j] : expf(-rate * softplus32(av[m][j] + bias[j])))
                        : head_decay;
                }
            }
        }
    };

    // ---- the four state warps
    const int col0_local = (warp % kRecWarps) * kRecColsPerWarp;
    const int col0 = blockIdx.z * kRecCols + col0_local;
    const int mine = 2 * ((lane >> 4) & 1) + ((lane >> 3) & 1);   // the column whose sums this lane gets
    // a head's matrix is stored column by column ([dv][dk]): a warp reads a column as one line
    float* st = state + (static_cast<size_t>(state_slot[r]) * heads + h) * dk * dv
        + static_cast<size_t>(col0) * dk;
    const bool runs = dk % V == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0;
    float s[kRecColsPerWarp][RL];
    if (!loader) {
#pragma unroll
        for (int c = 0; c < kRecColsPerWarp; ++c)
            rec_state_rows<R, false>(st + static_cast<size_t>(c) * dk, s[c], lane, dk, col0 + c < dv, runs);
    }
    auto advance = [&](int blk) {
        const float* buf = rec_smem + (blk & 1) * rec_buffer_floats(B, DP);
        const float* q_s = buf;
        const float* k_s = buf + B * DP;
        const float* g_s = buf + 2 * B * DP;
        const float* v_s = buf + 3 * B * DP;
        const float* b_s = v_s + B * kRecCols;
        const int t0 = first + blk * B;
        const int n_tok = min(B, last - t0);
        for (int tok = 0; tok < n_tok; ++tok) {
            float kk[RL], xx[RL], d[4], u[4];
            rec_load_rows<R>(g_s + tok * DP + lane * V, xx);
            rec_load_rows<R>(k_s + tok * DP + lane * V, kk);
#pragma unroll
            for (int c = 0; c < kRecColsPerWarp; ++c) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < RL; ++i) {
                    s[c][i] *= xx[i];
                    if (DELTA) acc = fmaf(s[c][i], kk[i], acc);
                }
                d[c] = acc;
            }
            if (DELTA) {
                const float dot = rec_reduce4(d, lane);
                rec_gather4(b_s[tok] * (v_s[tok * kRecCols + col0_local + mine] - dot), lane, u);
            } else {
                const float4 x = *reinterpret_cast<const float4*>(v_s + tok * kRecCols + col0_local);
                u[0] = x.x; u[1] = x.y; u[2] = x.z; u[3] = x.w;
            }
            rec_load_rows<R>(q_s + tok * DP + lane * V, xx);
#pragma unroll
            for (int c = 0; c < kRecColsPerWarp; ++c) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < RL; ++i) {
                    s[c][i] = fmaf(kk[i], u[c], s[c][i]);
                    acc = fmaf(s[c][i], xx[i], acc);
                }
                d[c] = acc;
            }
            const float o_sum = rec_reduce4(d, lane);
            if ((lane & 7) == 0 && col0 + mine < dv)
                y[static_cast<size_t>(t0 + tok) * heads * dv + static_cast<size_t>(h) * dv + col0 + mine] = o_sum;
        }
    };

    if (loader && blocks > 0) stage(0);
    __syncthreads();
    for (int blk = 0; blk < blocks; ++blk) {
        if (loader) {
            if (blk + 1 < blocks) stage(blk + 1);
        } else {
            advance(blk);
        }
        __syncthreads();                                   // block blk + 1 is staged, block blk is read
    }
    if (!loader) {
#pragma unroll
        for (int c = 0; c < kRecColsPerWarp; ++c)
            rec_state_rows<R, true>(st + static_cast<size_t>(c) * dk, s[c], lane, dk, col0 + c < dv, runs);
    }
}

// ------------------------------------------- rows of a long step, made ready once
// The CTAs of a head's column groups all need the same q, k and g of a row.  For a step of many
// rows this kernel computes them once, with the arithmetic of the scan's loaders in the same
// order (so the scan's result is the same bit for bit), and the scan's loaders only copy:
//     qn[t, qk head, :], kn[t, qk head, :]  activated and unit-normed, float32
//     gd[t, head, :] = exp(-exp(a_log) * softplus(a + dt_bias))          (a != null)
// A warp per (row, head); q and k are written by the first head of each query/key head's group.
constexpr int kRecPrepWarps = 4;
constexpr int kRecMaxPL = 8;                              // key widths up to 32 * kRecLanes

template <typename T>
__global__ void __launch_bounds__(kRecPrepWarps * 32)
matrix_state_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, long long q_stride,
                            long long k_stride, int act_silu, int unit, float unit_eps, float q_scale,
                            const float* __restrict__ a, long long a_stride,
                            const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                            float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ gd,
                            int rows, int heads, int qk_heads, int dk) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRecPrepWarps + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= rows) return;
    const int group = heads / qk_heads, qkh = h / group;
    const size_t row = static_cast<size_t>(t);
    if (a != nullptr) {
        const float rate = expf(a_log[h]);
#pragma unroll
        for (int j = 0; j < kRecMaxPL; ++j) {
            const int i = lane + 32 * j;
            if (i < dk) {
                const size_t c = static_cast<size_t>(h) * dk + i;
                gd[row * heads * dk + c] = expf(-rate * softplus32(a[row * a_stride + c] + dt_bias[c]));
            }
        }
    }
    if (h % group) return;
    float qv[kRecMaxPL], kv[kRecMaxPL];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int j = 0; j < kRecMaxPL; ++j) {
        const int i = lane + 32 * j;
        const bool in = i < dk;
        qv[j] = in ? to_float(q[row * q_stride + static_cast<size_t>(qkh) * dk + i]) : 0.f;
        kv[j] = in ? to_float(k[row * k_stride + static_cast<size_t>(qkh) * dk + i]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kRecMaxPL; ++j) {
        if (act_silu & 1) { qv[j] = silu32(qv[j]); kv[j] = silu32(kv[j]); }
        sq = fmaf(qv[j], qv[j], sq);
        sk = fmaf(kv[j], kv[j], sk);
    }
    float rq = q_scale, rk = 1.f;
    if (unit) {
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        rq = q_scale / sqrtf(sq + unit_eps);
        rk = 1.0f / sqrtf(sk + unit_eps);
    }
#pragma unroll
    for (int j = 0; j < kRecMaxPL; ++j) {
        const int i = lane + 32 * j;
        if (i < dk) {
            const size_t c = row * qk_heads * dk + static_cast<size_t>(qkh) * dk + i;
            qn[c] = qv[j] * rq;
            kn[c] = unit ? kv[j] * rk : kv[j];
        }
    }
}

// ------------------------------------------- RMS norm in parts, weight, sigmoid gate
// The C columns of y[t] in `groups` equal parts of n = C / groups, each divided by its own root
// mean square; out = that * weight[c % w_len] * sigmoid(gate[t, c]) (gate null: no gate; its rows
// lie `g_stride` elements apart; gate_act 1: SiLU of the gate instead of its sigmoid).  One CTA per (token, part).
template <typename TO>
__global__ void group_rmsnorm_gate_kernel(const float* __restrict__ y, const void* __restrict__ gate,
                                          int g_dtype, long long g_stride,
                                          const void* __restrict__ weight, int w_dtype, int w_len,
                                          float eps, TO* __restrict__ out, int C, int groups,
                                          int gate_act) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const int n = C / groups, c0 = part * n;
    const float* yr = y + static_cast<size_t>(t) * C + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
    TO* o = out + static_cast<size_t>(t) * C + c0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = yr[i] * r * load_as_float(weight, w_dtype, (c0 + i) % w_len);
        if (gate != nullptr) {
            const float g = load_as_float(gate, g_dtype, static_cast<size_t>(t) * g_stride + c0 + i);
            v *= gate_act == 1 ? silu32(g) : sigmoid32(g);
        }
        o[i] = from_float<TO>(v);
    }
}

// The same with a warp per (token, part), for parts of up to kPartWarpMax columns: a lane keeps
// its columns (lane + 32 j) in registers between the sum and the output.
constexpr int kPartWarpMax = 256;
constexpr int kPartWarps = 8;
template <typename TO>
__global__ void __launch_bounds__(kPartWarps * 32)
group_rmsnorm_gate_warp_kernel(const float* __restrict__ y, const void* __restrict__ gate, int g_dtype,
                               long long g_stride, const void* __restrict__ weight, int w_dtype,
                               int w_len, float eps, TO* __restrict__ out, int C, int groups,
                               long long parts, int gate_act) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long idx = static_cast<long long>(blockIdx.x) * kPartWarps + (threadIdx.x >> 5);
    if (idx >= parts) return;
    const long long t = idx / groups;
    const int part = static_cast<int>(idx - t * groups);
    const int n = C / groups, c0 = part * n;
    const float* yr = y + static_cast<size_t>(t) * C + c0;
    float v[kPartWarpMax / 32];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kPartWarpMax / 32; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < n ? yr[i] : 0.f;
        ss = fmaf(v[j], v[j], ss);
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
    TO* o = out + static_cast<size_t>(t) * C + c0;
#pragma unroll
    for (int j = 0; j < kPartWarpMax / 32; ++j) {
        const int i = lane + 32 * j;
        if (i < n) {
            float z = v[j] * r * load_as_float(weight, w_dtype, (c0 + i) % w_len);
            if (gate != nullptr) {
                const float g = load_as_float(gate, g_dtype, static_cast<size_t>(t) * g_stride + c0 + i);
                z *= gate_act == 1 ? silu32(g) : sigmoid32(g);
            }
            o[i] = from_float<TO>(z);
        }
    }
}

// ------------------------------------------- half the sum of two normed rows
// out[t] = 0.5 * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb), float32.  `a` and `b` may be
// float32 partial sums (`*_splits` slices `*_stride` apart, added in order).  One CTA per token;
// the two rows live in shared memory.
__global__ void rmsnorm_pair_mean_kernel(const void* __restrict__ a, int a_dtype, int a_splits,
                                         long long a_stride, const void* __restrict__ b, int b_dtype,
                                         int b_splits, long long b_stride,
                                         const void* __restrict__ wa, const void* __restrict__ wb,
                                         int w_dtype, float eps, float* __restrict__ out, int H) {
    extern __shared__ float pair_rows[];                  // a [H], b [H]
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = static_cast<size_t>(blockIdx.x) * H;
    float* ra_s = pair_rows;
    float* rb_s = pair_rows + H;
    float sa = 0.f, sb = 0.f;
    // partial sums are float32: their loads carry no branch on the type, so several are in flight
    auto value = [](const void* p, int dtype, int splits, long long stride, size_t idx) {
        if (dtype != SOMI_F32) return load_as_float(p, dtype, idx);
        const float* f = static_cast<const float*>(p) + idx;
        float x = f[0];
#pragma unroll 8
        for (int s = 1; s < splits; ++s) x += f[static_cast<size_t>(s) * stride];
        return x;
    };
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = value(a, a_dtype, a_splits, a_stride, base + i);
        const float z = value(b, b_dtype, b_splits, b_stride, base + i);
        ra_s[i] = x;
        rb_s[i] = z;
        sa = fmaf(x, x, sa);
        sb = fmaf(z, z, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / static_cast<float>(H) + eps);
    const float rb = 1.0f / sqrtf(sb / static_cast<float>(H) + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = ra_s[i] * ra * load_as_float(wa, w_dtype, i);
        const float z = rb_s[i] * rb * load_as_float(wb, w_dtype, i);
        out[base + i] = 0.5f * (x + z);
    }
}

// ---------------------------------------------------------------- relu squared
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float z = fmaxf(to_float(x[i]), 0.f);
        out[i] = from_float<T>(z * z);
    }
}

}  // namespace somi

using namespace somi;

static inline int threads_for(int n) { return min(256, max(32, ((n + 31) / 32) * 32)); }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

SOMI_API int somi_add_scaled_rmsnorm(float* residual, const void* a, int a_dtype, int a_splits,
                                     long long a_stride, const void* scale_a, const void* b,
                                     int b_dtype, int b_splits, long long b_stride,
                                     const void* scale_b, int scale_dtype, float mult,
                                     const float* extra, const void* w1, const void* w2, int w_dtype, float eps, void* out1, void* out2,
                                     int out_dtype, const int* rows, int n_out, int H, int write_back,
                                     cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if ((a_splits > 1 && a_dtype != SOMI_F32) || (b_splits > 1 && b_dtype != SOMI_F32))
        return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * H;
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    const int vec4 = (H & 3) == 0 && aligned16(residual) && aligned16(a) && aligned16(b) &&
                     aligned16(scale_a) && aligned16(scale_b) && aligned16(extra) && (a_stride & 3) == 0 &&
                     (b_stride & 3) == 0;
    const int threads = vec4 ? min(1024, max(32, (((n_out <= 512 ? H / 4 : H / 16) + 31) / 32) * 32))
                             : threads_for(H / 2);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(add_scaled_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    launch_pdl(add_scaled_rmsnorm_kernel, dim3(n_out), dim3(threads), smem, stream, residual, a,
               a_dtype, a_splits, a_stride, scale_a, b, b_dtype, b_splits, b_stride, scale_b,
               scale_dtype, mult, extra, w1, w2, w_dtype, eps, out1, out2, out_dtype, rows, H,
               write_back, vec4);
    return launch_status();
}

SOMI_API int somi_headnorm_rotary_store(void* qkv, int dtype, long long stride, const int* positions,
                                        const double* inv_freq, int T, int nq, int nkv, int hd, int vd,
                                        int rot, const void* q_w, const void* k_w, int w_dtype,
                                        float eps, float magnitude, const int* slot_map, void* kcache,
                                        void* vcache, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > 1024 || vd <= 0 || rot < 0 || rot > hd || (rot & 1) || nq <= 0 || nkv <= 0)
        return SOMI_ERR_UNSUPPORTED;
    const int warps = min(8, nq + nkv);
    const dim3 grid(T, T <= 256 ? (nq + nkv + 7) / 8 : 1);
    const size_t smem = sizeof(float) * warps * hd;
    if (dtype == SOMI_F32)
        launch_pdl(headnorm_rotary_store_kernel<float>, grid, dim3(32 * warps), smem, stream,
                   static_cast<float*>(qkv), stride, positions, inv_freq, nq, nkv, hd, vd, rot, q_w,
                   k_w, w_dtype, eps, magnitude, slot_map, static_cast<float*>(kcache),
                   static_cast<float*>(vcache), page_size);
    else
        launch_pdl(headnorm_rotary_store_kernel<__nv_bfloat16>, grid, dim3(32 * warps), smem, stream,
                   static_cast<__nv_bfloat16*>(qkv), stride, positions, inv_freq, nq, nkv, hd, vd,
                   rot, q_w, k_w, w_dtype, eps, magnitude, slot_map, static_cast<__nv_bfloat16*>(kcache),
                   static_cast<__nv_bfloat16*>(vcache), page_size);
    return launch_status();
}

SOMI_API int somi_matrix_state_scan_max_key() { return 32 * kRecLanes; }

// q, k: [T, *_stride] with qk_heads heads of dk elements from the pointer on; v: heads heads of dv.
// delta != 0: beta [T, beta_stride] logits per head, of q's dtype.  a != null: float32 [T, a_stride]
// decay logits per head and key channel with dt_bias [heads * dk] and a_log [heads]; else
// decay [heads] (decay_ready: a holds the decays).  dtype: of q and k; vb_dtype: of v and beta.
// state: float32 [slots, heads, dv, dk]; y: float32 [T, heads * dv].  max_rows: the
// most rows any request has in this step (0: not known); it only chooses how many rows are staged
// at a time, the sums are the same.
SOMI_API int somi_matrix_state_scan(const void* q, const void* k, const void* v, int dtype,
                                    int vb_dtype, long long q_stride, long long k_stride,
                                    long long v_stride, int act_silu, int unit, float unit_eps,
                                    float q_scale, int delta, const void* beta, long long beta_stride,
                                    const float* a, long long a_stride, int decay_ready,
                                    const float* dt_bias, const float* a_log,
                                    const float* decay, float* state, const int* cu_q,
                                    const int* state_slot, float* y, int R, int heads, int qk_heads,
                                    int dk, int dv, int max_rows, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (dk <= 0 || dk > 32 * kRecLanes || dv <= 0 || heads <= 0 || qk_heads <= 0 || heads % qk_heads ||
        (delta && beta == nullptr) || (a == nullptr && decay == nullptr) ||
        (a != nullptr && (dt_bias == nullptr || a_log == nullptr)))
        return SOMI_ERR_UNSUPPORTED;
    dim3 grid(R, heads, (dv + kRecCols - 1) / kRecCols);
    const int rows = (dk + kRecLanes - 1) / kRecLanes;
#define SOMI_LAUNCH_REC_B(TT, RR, DD, BB)                                                         \
    const size_t smem = sizeof(float) * 2 * rec_buffer_floats(BB, RR * kRecLanes);                \
    if (smem > 48 * 1024)                                                                         \
        cudaFuncSetAttribute(matrix_state_scan_kernel<TT, RR, DD, BB>,                            \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
    launch_pdl(matrix_state_scan_kernel<TT, RR, DD, BB>, grid, dim3(kRecThreads), smem, stream,   \
               static_cast<const TT*>(q), static_cast<const TT*>(k), v, vb_dtype,                 \
               q_stride, k_stride, v_stride, act_silu, unit, unit_eps, q_scale,                 \
               beta, beta_stride, a, a_stride, decay_ready, dt_bias, a_log, decay, state, cu_q, state_slot, y, heads, qk_heads, dk, dv)
    // short steps stage little, so that more CTAs are resident while their states stream in
#define SOMI_LAUNCH_REC(TT, RR, DD)                                                               \
    if (max_rows > 0 && max_rows <= kRecBlockShort) { SOMI_LAUNCH_REC_B(TT, RR, DD, kRecBlockShort); } \
    else { SOMI_LAUNCH_REC_B(TT, RR, DD, kRecBlockLong); }
#define SOMI_REC_BY_ROWS(TT, DD)                                                                  \
    do {                                                                                          \
        if (rows <= 4) { SOMI_LAUNCH_REC(TT, 4, DD); }                                       \
        else if (rows <= 8) { SOMI_LAUNCH_REC(TT, 8, DD); }                                       \
        else if (rows <= 16) { SOMI_LAUNCH_REC(TT, 16, DD); }                                     \
        else { SOMI_LAUNCH_REC(TT, 32, DD); }                                                     \
    } while (0)
    if (dtype == SOMI_F32) {
        if (delta) SOMI_REC_BY_ROWS(float, true);
        else SOMI_REC_BY_ROWS(float, false);
    } else {
        if (delta) SOMI_REC_BY_ROWS(__nv_bfloat16, true);
        else SOMI_REC_BY_ROWS(__nv_bfloat16, false);
    }
#undef SOMI_REC_BY_ROWS
#undef SOMI_LAUNCH_REC
#undef SOMI_LAUNCH_REC_B
    return launch_status();
}

// q, k: [T, *_stride] of `dtype` -> qn, kn: float32 [T, qk_heads * dk]; a (may be null) ->
// gd: float32 [T, heads * dk].  See matrix_state_prepare_kernel.
SOMI_API int somi_matrix_state_prepare(const void* q, const void* k, int dtype, long long q_stride,
                                       long long k_stride, int act_silu, int unit, float unit_eps,
                                       float q_scale, const float* a, long long a_stride,
                                       const float* dt_bias, const float* a_log, float* qn, float* kn,
                                       float* gd, int T, int heads, int qk_heads, int dk,
                                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dk <= 0 || dk > 32 * kRecMaxPL || heads <= 0 || qk_heads <= 0 || heads % qk_heads ||
        (a != nullptr && (dt_bias == nullptr || a_log == nullptr || gd == nullptr)))
        return SOMI_ERR_UNSUPPORTED;
    const dim3 grid((T + kRecPrepWarps - 1) / kRecPrepWarps, heads);
    if (dtype == SOMI_F32)
        launch_pdl(matrix_state_prepare_kernel<float>, grid, dim3(kRecPrepWarps * 32), 0, stream,
                   static_cast<const float*>(q), static_cast<const float*>(k), q_stride, k_stride,
                   act_silu, unit, unit_eps, q_scale, a, a_stride, dt_bias, a_log, qn, kn, gd, T, heads,
                   qk_heads, dk);
    else
        launch_pdl(matrix_state_prepare_kernel<__nv_bfloat16>, grid, dim3(kRecPrepWarps * 32), 0, stream,
                   static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), q_stride,
                   k_stride, act_silu, unit, unit_eps, q_scale, a, a_stride, dt_bias, a_log, qn, kn, gd,
                   T, heads, qk_heads, dk);
    return launch_status();
}

SOMI_API int somi_group_rmsnorm_gate(const float* y, const void* gate, int g_dtype, long long g_stride,
                                     const void* weight, int w_dtype, int w_len, float eps, void* out,
                                     int out_dtype, int T, int C, int groups, int gate_act,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (groups <= 0 || C % groups || w_len <= 0) return SOMI_ERR_UNSUPPORTED;
    const int threads = threads_for(C / groups);
    if (C / groups <= kPartWarpMax) {                     // short parts: a warp each
        const long long parts = static_cast<long long>(T) * groups;
        const dim3 grid(static_cast<unsigned>((parts + kPartWarps - 1) / kPartWarps));
        if (out_dtype == SOMI_F32)
            launch_pdl(group_rmsnorm_gate_warp_kernel<float>, grid, dim3(kPartWarps * 32), 0, stream, y,
                       gate, g_dtype, g_stride, weight, w_dtype, w_len, eps, static_cast<float*>(out), C,
                       groups, parts, gate_act);
        else
            launch_pdl(group_rmsnorm_gate_warp_kernel<__nv_bfloat16>, grid, dim3(kPartWarps * 32), 0,
                       stream, y, gate, g_dtype, g_stride, weight, w_dtype, w_len, eps,
                       static_cast<__nv_bfloat16*>(out), C, groups, parts, gate_act);
        return launch_status();
    }
    if (out_dtype == SOMI_F32)
        launch_pdl(group_rmsnorm_gate_kernel<float>, dim3(T, groups), dim3(threads), 0, stream, y, gate,
                   g_dtype, g_stride, weight, w_dtype, w_len, eps, static_cast<float*>(out), C, groups,
                   gate_act);
    else
        launch_pdl(group_rmsnorm_gate_kernel<__nv_bfloat16>, dim3(T, groups), dim3(threads), 0, stream,
                   y, gate, g_dtype, g_stride, weight, w_dtype, w_len, eps,
                   static_cast<__nv_bfloat16*>(out), C, groups, gate_act);
    return launch_status();
}

SOMI_API int somi_rmsnorm_pair_mean(const void* a, int a_dtype, int a_splits, long long a_stride,
                                    const void* b, int b_dtype, int b_splits, long long b_stride,
                                    const void* wa, const void* wb, int w_dtype, float eps,
                                    float* out, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if ((a_splits > 1 && a_dtype != SOMI_F32) || (b_splits > 1 && b_dtype != SOMI_F32))
        return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * 2 * H;
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(rmsnorm_pair_mean_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    const int threads = min(1024, max(32, ((H / 4 + 31) / 32) * 32));
    launch_pdl(rmsnorm_pair_mean_kernel, dim3(T), dim3(threads), smem, stream, a, a_dtype,
               a_splits, a_stride, b, b_dtype, b_splits, b_stride, wa, wb, w_dtype, eps, out, H);
    return launch_status();
}

SOMI_API int somi_relu2(const void* x, void* out, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = static_cast<int>(((n + 255) / 256) < 148LL * 16 ? ((n + 255) / 256) : 148LL * 16);
    if (dtype == SOMI_F32)
        launch_pdl(relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const float*>(x), static_cast<float*>(out), n);
    else
        launch_pdl(relu2_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n);
    return launch_status();
}
