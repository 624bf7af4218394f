// Causal grouped-query attention over the paged cache, any dtype, any key and value width up
// to 256, any page size: the reference kernel of the library.  Which earlier keys a token sees
// is a parameter: all of them, the last `window`, or those of its own chunk (positions
// i and j with i / chunk == j / chunk, chunks counted from position 0 of the sequence).  The
// output may be multiplied by sigmoid(gate) in the epilogue (a logit per output element, or with
// `gate_per_head` one per token and head).  `softcap` > 0: a score s becomes
// softcap * tanh(s / softcap) before the softmax.  `sinks`: a score per query head that joins the
// softmax's denominator without a key or a value (0 gives "one more in the denominator").
// It is the float32 path's attention and the fallback of the bfloat16 path for
// sizes that the tensor-core kernels refuse.  Products are accumulated with
// float32 FMAs, softmax is float32 and online, key tiles are aligned to
// multiples of BN from position 0, so the arithmetic on one query row does not
// depend on how its request was cut into steps or on what else is in the batch.
//
// One CTA = one q tile (<= BM consecutive tokens of one request) x one query head.
// Tiles [0, n_tiles) come from the tile list (request, first row, rows); CTAs
// beyond them are the single-token requests: request n_prefill_req + i, row
// n_prefill_tok + i.
#include "common.cuh"

namespace somi {

constexpr int kBM = 16;        // query rows per CTA
constexpr int kBN = 32;        // keys per iteration
constexpr int kThreads = 128;
constexpr int kMaxHd = 256;
constexpr int kAccPerThread = kBM * kMaxHd / kThreads;   // 32

template <typename T>
__global__ void __launch_bounds__(kThreads)
paged_attention_generic_kernel(const T* __restrict__ qkv, int row_stride,
                               const T* __restrict__ kcache, const T* __restrict__ vcache,
                               const int* __restrict__ block_table, int bt_stride,
                               const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                               const int* __restrict__ tiles, int n_tiles, int n_prefill_req,
                               int n_prefill_tok, int nq, int nkv, int hd, int vd, int page_size,
                               float scale, int window, int chunk, const T* __restrict__ gate,
                               long long gate_stride, int gate_per_head, float softcap,
                               const float* __restrict__ sinks, T* __restrict__ out) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    float* Qs = smem;                           // [kBM][hd]
    float* Ks = Qs + kBM * hd;                  // [kBN][hd + 1]
    float* Vs = Ks + kBN * (hd + 1);            // [kBN][vd]
    float* Ss = Vs + kBN * vd;                  // [kBM][kBN + 1]
    float* m_s = Ss + kBM * (kBN + 1);          // [kBM]
    float* l_s = m_s + kBM;                     // [kBM]
    float* a_s = l_s + kBM;                     // [kBM]

    int req, row0, rows;
    if (static_cast<int>(blockIdx.x) < n_tiles) {
        req = tiles[3 * blockIdx.x];
        row0 = tiles[3 * blockIdx.x + 1];
        rows = tiles[3 * blockIdx.x + 2];
    } else {
        const int i = blockIdx.x - n_tiles;
        req = n_prefill_req + i;
        row0 = n_prefill_tok + i;
        rows = 1;
    }
    const int head = blockIdx.y;
    const int kvh = head / (nq / nkv);
    const int tid = threadIdx.x;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;                                   // exclusive
    // first key any row reads
    const int kv_first = chunk > 0 ? (q_pos0 / chunk) * chunk : (window > 0 ? max(0, q_pos0 - window + 1) : 0);
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    for (int idx = tid; idx < kBM * hd; idx += kThreads) {
        const int m = idx / hd, d = idx - m * hd;
        Qs[idx] = m < rows ? to_float(qkv[static_cast<size_t>(row0 + m) * row_stride + head * hd + d]) * scale
                           : 0.f;
    }
    if (tid < kBM) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    float acc[kAccPerThread];
#pragma unroll
    for (int i = 0; i < kAccPerThread; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int kb = (kv_first / kBN) * kBN; kb < kv_end; kb += kBN) {
        for (int idx = tid; idx < kBN * hd; idx += kThreads) {
            const int n = idx / hd, d = idx - n * hd;
            const int j = kb + n;
            float kval = 0.f;
            if (j >= kv_first && j < kv_end) {
                const int page = bt[j / page_size];
                kval = to_float(kcache[((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * hd + d]);
            }
            Ks[n * (hd + 1) + d] = kval;
        }
        for (int idx = tid; idx < kBN * vd; idx += kThreads) {
            const int n = idx / vd, d = idx - n * vd;
            const int j = kb + n;
            float vval = 0.f;
            if (j >= kv_first && j < kv_end) {
                const int page = bt[j / page_size];
                vval = to_float(vcache[((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * vd + d]);
            }
            Vs[n * vd + d] = vval;
        }
        __syncthreads();
        for (int idx = tid; idx < kBM * kBN; idx += kThreads) {
            const int m = idx / kBN, n = idx - m * kBN;
            const int j = kb + n, qp = q_pos0 + m;
            float s = -INFINITY;
            if (m < rows && j <= qp && j >= kv_first && (window <= 0 || j > qp - window) &&
                (chunk <= 0 || j / chunk == qp / chunk)) {
                s = 0.f;
                const float* q = Qs + m * hd;
                const float* k = Ks + n * (hd + 1);
                for (int d = 0; d < hd; ++d) s = fmaf(q[d], k[d], s);
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            }
            Ss[m * (kBN + 1) + n] = s;
        }
        __syncthreads();
        {   // online softmax: one warp per row, one key per lane (kBN == 32)
            const int warp = tid >> 5, lane = tid & 31;
            for (int m = warp; m < kBM; m += kThreads / 32) {
                const float s = Ss[m * (kBN + 1) + lane];
                const float m_old = m_s[m];
                const float m_new = fmaxf(m_old, warp_max(s));
                float p = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    alpha = expf(m_old - m_new);          // m_old = -inf gives 0
                    p = expf(s - m_new);                   // s = -inf gives 0
                }
                const float psum = warp_sum(p);
                Ss[m * (kBN + 1) + lane] = p;
                if (lane == 0) {
                    m_s[m] = m_new;
                    l_s[m] = l_s[m] * alpha + psum;
                    a_s[m] = alpha;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kAccPerThread; ++i) {
            const int idx = tid + i * kThreads;
            if (idx < kBM * vd) {
                const int m = idx / vd, d = idx - m * vd;
                float o = acc[i] * a_s[m];
                const float* p = Ss + m * (kBN + 1);
                for (int n = 0; n < kBN; ++n) o = fmaf(p[n], Vs[n * vd + d], o);
                acc[i] = o;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < kAccPerThread; ++i) {
        const int idx = tid + i * kThreads;
        if (idx < kBM * vd) {
            const int m = idx / vd, d = idx - m * vd;
            if (m < rows) {
                float den = l_s[m];
                if (sinks != nullptr) den += expf(sinks[head] - m_s[m]);
                float o = acc[i] / den;
                if (gate != nullptr) {
                    const float z = to_float(gate[static_cast<size_t>(row0 + m) * gate_stride +
                                                  (gate_per_head ? head : head * vd + d)]);
                    o = o / (1.0f + expf(-z));
                }
                out[static_cast<size_t>(row0 + m) * (nq * vd) + head * vd + d] = from_float<T>(o);
            }
        }
    }
}

// x[t, h * vd + d] *= sigmoid(gate[t * gate_stride + h]): one logit per token and head, for the
// attention kernels that leave the gate to a kernel of its own.
template <typename T>
__global__ void head_gate_mul_kernel(T* __restrict__ x, const T* __restrict__ gate, long long gate_stride,
                                     int heads, int vd, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    const long long per_row = static_cast<long long>(heads) * vd;
    if (sizeof(T) == 2 && (vd & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // eight neighbours of one head a thread: one 16-byte access, one sigmoid
        for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
            const long long t = i / per_row;
            const int h = static_cast<int>((i - t * per_row) / vd);
            const float g = 1.0f / (1.0f + expf(-to_float(gate[t * gate_stride + h])));
            uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + i);
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                v[e] = __floats2bfloat162_rn(__low2float(v[e]) * g, __high2float(v[e]) * g);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(x) + i) = raw;
        }
        return;
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / per_row;
        const int h = static_cast<int>((i - t * per_row) / vd);
        const float z = to_float(gate[t * gate_stride + h]);
        x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-z)));
    }
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_head_gate_mul(void* x, const void* gate, int dtype, long long gate_stride,
                                long long rows, int heads, int vd, cudaStream_t stream) {
    const long long n = rows * heads * vd;
    if (n <= 0) return 0;
    const long long work = dtype == SOMI_F32 ? n : (n + 7) / 8;
    const int blocks = static_cast<int>(((work + 255) / 256) < 148LL * 16 ? ((work + 255) / 256) : 148LL * 16);
    if (dtype == SOMI_F32)
        launch_pdl(head_gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<float*>(x), static_cast<const float*>(gate), gate_stride, heads, vd, n);
    else
        launch_pdl(head_gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gate),
                   gate_stride, heads, vd, n);
    return launch_status();
}

SOMI_API int somi_attention_generic_q_tile() { return kBM; }

SOMI_API int somi_paged_attention_generic(
    const void* qkv, int dtype, int row_stride, const void* kcache, const void* vcache,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int n_prefill_req, int n_prefill_tok, int n_decode, int nq, int nkv, int hd, int vd,
    int page_size, float scale, int window, int chunk, const void* gate, long long gate_stride,
    int gate_per_head, float softcap, const float* sinks, void* out, cudaStream_t stream) {
    if (n_tiles + n_decode <= 0) return 0;
    if (hd <= 0 || hd > kMaxHd || vd <= 0 || vd > kMaxHd || nkv <= 0 || nq % nkv || page_size <= 0 ||
        (window > 0 && chunk > 0))
        return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kBM) * hd + kBN * (hd + 1) + kBN * vd +
                                         kBM * (kBN + 1) + 3 * kBM);
    dim3 grid(n_tiles + n_decode, nq);
#define SOMI_LAUNCH_ATT(T)                                                                      \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(paged_attention_generic_kernel<T>,                             \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        launch_pdl(paged_attention_generic_kernel<T>, dim3(grid), dim3(kThreads), smem, stream,                     \
            static_cast<const T*>(qkv), row_stride, static_cast<const T*>(kcache),              \
            static_cast<const T*>(vcache), block_table, bt_stride, cu_q, ctx_len, tiles,        \
            n_tiles, n_prefill_req, n_prefill_tok, nq, nkv, hd, vd, page_size, scale, window,   \
            chunk, static_cast<const T*>(gate), gate_stride, gate_per_head, softcap, sinks,     \
            static_cast<T*>(out));                                                              \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_ATT(float);
    else SOMI_LAUNCH_ATT(__nv_bfloat16);
#undef SOMI_LAUNCH_ATT
    return launch_status();
}
