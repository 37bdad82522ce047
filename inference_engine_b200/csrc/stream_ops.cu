// Operations on the residual stream and around it that models with hashed bigram embeddings,
// norms on both sides of a sublayer, biased gated feed-forwards and re-injected embeddings need:
//
//  * bigram_embedding: out[n] = embed[id] + bigram[row], row = (prev * mul_prev + id * mul_cur) mod
//    buckets, or row `buckets` for a request's first token.  The token before a step's first one is
//    kept per request in a state slot (as the integer's bits) and moved on by the same block that
//    read it.
//  * sandwich_norm: y = sum of the parts of `delta` (+ the parts of `delta2`, the output of a second
//    sublayer that read the same input) (+ bias) (+ the row of `extra`, a second stream of the rows'
//    shape: the embedding's output that a looped model adds again); y <- rms(y) * post_w (if post_w);
//    h += y; out = rms(h) * pre_w (if out).  One block per row; both sums of squares are added in
//    an order that depends on the row's width alone.
//  * silu_mul_bias: out = silu(g + bg) * (u + bu) from rows that hold gates, then ups (32-bit, or the
//    compute dtype); biases and activation in 32-bit.
//  * gated_add_norm: h += sigmoid(gate_pre + gate_bias) * (sum of the parts of `delta`), element by
//    element (a model whose sublayers enter the residual stream through a learned gate);
//    out = rms(h) * w (if out).  One block per row, sums in an order that depends on the width alone.
//  * polynorm: out = a N(z) + b N(z^2) + c N(z^3) + e per row, powers element by element,
//    N(y) = y / sqrt(mean(y^2) + eps) over the row; sums and powers in 32-bit.
//  * concat_cast: out[n] = [h[n]; x0[n]] in the compute dtype.
//  * weighted_sum: out = sa * a + sb * b (32-bit).
#include "common.cuh"
#include <math.h>

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
bigram_embedding_kernel(const T* __restrict__ embed, const T* __restrict__ bigram, const int* __restrict__ ids,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ cu_q, const int* __restrict__ slots, int* __restrict__ state,
                        long long state_stride, int num_slots, float* __restrict__ out, int hidden, int vocab,
                        int buckets, long long mul_prev, long long mul_cur, int* err) {
    __shared__ int s_row;
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) ie_report(err, IE_ERR_TOKEN_ID, id, n);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)n * hidden + i] = 0.f;
        return;
    }
    if (threadIdx.x == 0) {
        int seq = seq_of_token[n], first = cu_q[seq], end = cu_q[seq + 1];
        int slot = slots[seq];
        bool slot_ok = slot >= 0 && slot < num_slots;
        int row = buckets;
        if (positions[n] > 0) {
            int prev = 0;
            if (n > first) prev = ids[n - 1];
            else if (slot_ok) prev = state[(size_t)slot * state_stride];
            else ie_report(err, IE_ERR_PAGE, slot, n);
            row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets);
            if (row < 0) row += buckets;
        }
        // the request's last token of this step is what its next step starts from; the block of the
        // request's first token is the only one that touches the slot, after it has read it
        if (n == first && end > first && slot_ok) state[(size_t)slot * state_stride] = ids[end - 1];
        s_row = row;
    }
    __syncthreads();
    const T* e = embed + (size_t)id * hidden;
    const T* b = bigram + (size_t)s_row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)n * hidden + i] = ie_load(e + i) + ie_load(b + i);
}

constexpr int SN_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();  // (red may still be read from the sum before)
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < SN_THREADS / 32; ++w) total += red[w];
    return total;
}

template <int VEC>
struct Pack { float v[VEC]; };
template <int VEC>
__device__ __forceinline__ Pack<VEC> load_pack(const float* p) {
    Pack<VEC> r;
    if (VEC == 4) {
        float4 t = *reinterpret_cast<const float4*>(p);
        r.v[0] = t.x; r.v[1 % VEC] = t.y; r.v[2 % VEC] = t.z; r.v[3 % VEC] = t.w;
    } else {
        r.v[0] = *p;
    }
    return r;
}
template <int VEC>
__device__ __forceinline__ void store_pack(float* p, const Pack<VEC>& r) {
    if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1 % VEC], r.v[2 % VEC], r.v[3 % VEC]);
    else *p = r.v[0];
}
template <int VEC>
__device__ __forceinline__ void store_pack(__nv_bfloat16* p, const Pack<VEC>& r) {
    if (VEC == 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1 % VEC]), hi = __floats2bfloat162_rn(r.v[2 % VEC], r.v[3 % VEC]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
    } else {
        *p = __float2bfloat16_rn(r.v[0]);
    }
}

// VEC = 4: rows whose width is a multiple of 4 move as 16-byte pieces (the sums are taken in the same
// order for a given width either way: a thread adds its entries in rising order, then the block adds).
template <typename OutT, int VEC>
__global__ void __launch_bounds__(SN_THREADS)
sandwich_norm_kernel(float* __restrict__ h, const float* __restrict__ delta, int num_partials, size_t partial_stride,
                     const float* __restrict__ delta2, int num_partials2, size_t partial_stride2,
                     const float* __restrict__ extra, const float* __restrict__ bias, const float* __restrict__ post_w, float post_eps,
                     const float* __restrict__ pre_w, float pre_eps, OutT* __restrict__ out,
                     const int* __restrict__ rows, int hidden) {
    extern __shared__ __align__(16) float row_buf[];  // [hidden]
    __shared__ float red[SN_THREADS / 32];
    ie_pdl_trigger();
    ie_pdl_wait();
    int r = blockIdx.x;
    size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    if (delta != nullptr) {
        for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
            Pack<VEC> y = load_pack<VEC>(delta + src + i);
            for (int p = 1; p < num_partials; ++p) {
                Pack<VEC> d = load_pack<VEC>(delta + p * partial_stride + src + i);
#pragma unroll
                for (int v = 0; v < VEC; ++v) y.v[v] += d.v[v];
            }
            for (int p = 0; p < num_partials2; ++p) {
                Pack<VEC> d = load_pack<VEC>(delta2 + p * partial_stride2 + src + i);
#pragma unroll
                for (int v = 0; v < VEC; ++v) y.v[v] += d.v[v];
            }
            if (extra) {
                Pack<VEC> d = load_pack<VEC>(extra + src + i);
#pragma unroll
                for (int v = 0; v < VEC; ++v) y.v[v] += d.v[v];
            }
            if (bias) {
                Pack<VEC> b = load_pack<VEC>(bias + i);
#pragma unroll
                for (int v = 0; v < VEC; ++v) y.v[v] += b.v[v];
            }
            store_pack<VEC>(row_buf + i, y);
#pragma unroll
            for (int v = 0; v < VEC; ++v) ss = fmaf(y.v[v], y.v[v], ss);
        }
        float inv = 1.0f;
        if (post_w != nullptr) inv = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + post_eps);
        ss = 0.f;
        for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
            Pack<VEC> y = load_pack<VEC>(row_buf + i), x = load_pack<VEC>(h + src + i);
            if (post_w != nullptr) {
                Pack<VEC> w = load_pack<VEC>(post_w + i);
#pragma unroll
                for (int v = 0; v < VEC; ++v) y.v[v] = w.v[v] * (y.v[v] * inv);
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                x.v[v] += y.v[v];
                ss = fmaf(x.v[v], x.v[v], ss);
            }
            store_pack<VEC>(row_buf + i, x);
            if (rows == nullptr) store_pack<VEC>(h + src + i, x);
        }
    } else {
        for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
            Pack<VEC> x = load_pack<VEC>(h + src + i);
            store_pack<VEC>(row_buf + i, x);
#pragma unroll
            for (int v = 0; v < VEC; ++v) ss = fmaf(x.v[v], x.v[v], ss);
        }
    }
    if (out == nullptr) return;
    float inv2 = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + pre_eps);
    for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
        Pack<VEC> x = load_pack<VEC>(row_buf + i), w = load_pack<VEC>(pre_w + i);
#pragma unroll
        for (int v = 0; v < VEC; ++v) x.v[v] = w.v[v] * (x.v[v] * inv2);
        store_pack<VEC>(out + (size_t)r * hidden + i, x);
    }
}

__device__ __forceinline__ float sigmoid_precise(float z) { return 1.0f / (1.0f + expf(-z)); }

// gate_pre: [N, hidden] 32-bit (rows as in h, `gate_ld` numbers apart: it may be some columns of a wider
// product), or `gate_partials` such arrays `gate_stride` apart, the parts of a split product, added in
// order; gate_bias: [hidden] or null.  `rows` selects rows and
// leaves h as it is; out == null: only h is brought up to date.
template <typename OutT, int VEC>
__global__ void __launch_bounds__(SN_THREADS)
gated_add_norm_kernel(float* __restrict__ h, const float* __restrict__ delta, int num_partials, size_t partial_stride,
                      const float* __restrict__ gate_pre, int gate_partials, size_t gate_stride, int gate_ld,
                      const float* __restrict__ gate_bias, const float* __restrict__ weight, float eps,
                      OutT* __restrict__ out, const int* __restrict__ rows, int hidden) {
    extern __shared__ __align__(16) float row_buf[];  // [hidden]
    __shared__ float red[SN_THREADS / 32];
    ie_pdl_trigger();
    ie_pdl_wait();
    int r = blockIdx.x;
    size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    size_t gsrc = (size_t)(rows ? rows[r] : r) * gate_ld;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
        Pack<VEC> y = load_pack<VEC>(delta + src + i);
        for (int p = 1; p < num_partials; ++p) {
            Pack<VEC> d = load_pack<VEC>(delta + p * partial_stride + src + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) y.v[v] += d.v[v];
        }
        Pack<VEC> g = load_pack<VEC>(gate_pre + gsrc + i), x = load_pack<VEC>(h + src + i);
        for (int p = 1; p < gate_partials; ++p) {
            Pack<VEC> d = load_pack<VEC>(gate_pre + p * gate_stride + gsrc + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) g.v[v] += d.v[v];
        }
        if (gate_bias != nullptr) {
            Pack<VEC> b = load_pack<VEC>(gate_bias + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) g.v[v] += b.v[v];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            x.v[v] = fmaf(sigmoid_precise(g.v[v]), y.v[v], x.v[v]);
            ss = fmaf(x.v[v], x.v[v], ss);
        }
        store_pack<VEC>(row_buf + i, x);
        if (rows == nullptr) store_pack<VEC>(h + src + i, x);
    }
    if (out == nullptr) return;
    float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    for (int i = threadIdx.x * VEC; i < hidden; i += SN_THREADS * VEC) {
        Pack<VEC> x = load_pack<VEC>(row_buf + i), w = load_pack<VEC>(weight + i);
#pragma unroll
        for (int v = 0; v < VEC; ++v) x.v[v] = w.v[v] * (x.v[v] * inv);
        store_pack<VEC>(out + (size_t)r * hidden + i, x);
    }
}

// One block per row of `z` ([N, width], rows `z_ld` numbers apart, 32-bit or the compute dtype); coeff: a, b, c, e.
template <typename InT, typename OutT>
__global__ void __launch_bounds__(SN_THREADS)
polynorm_kernel(const InT* __restrict__ z, int z_ld, const float* __restrict__ coeff, float eps,
                OutT* __restrict__ out, int width) {
    extern __shared__ __align__(16) float row_buf[];  // [width]
    __shared__ float red[SN_THREADS / 32];
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t at = (size_t)blockIdx.x * width, z_at = (size_t)blockIdx.x * z_ld;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < width; i += SN_THREADS) {
        float x = ie_load(z + z_at + i), x2 = x * x, x3 = x2 * x;
        row_buf[i] = x;
        s2 += x2;
        s4 = fmaf(x2, x2, s4);
        s6 = fmaf(x3, x3, s6);
    }
    float n = (float)width;
    float r1 = 1.0f / sqrtf(block_sum(s2, red) / n + eps);
    float r2 = 1.0f / sqrtf(block_sum(s4, red) / n + eps);
    float r3 = 1.0f / sqrtf(block_sum(s6, red) / n + eps);
    float a = coeff[0] * r1, b = coeff[1] * r2, c = coeff[2] * r3, e = coeff[3];
    for (int i = threadIdx.x; i < width; i += SN_THREADS) {
        float x = row_buf[i];
        ie_store(out + at + i, fmaf(x, fmaf(x, fmaf(x, c, b), a), e));
    }
}

template <typename T, typename InT>
__global__ void silu_mul_bias_kernel(const InT* __restrict__ gate_up, const float* __restrict__ bias,
                                     T* __restrict__ out, int inter, size_t total) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        size_t row = idx / inter;
        int i = (int)(idx - row * inter);
        float g = ie_load(gate_up + row * 2 * inter + i), u = ie_load(gate_up + row * 2 * inter + inter + i);
        if (bias) { g += bias[i]; u += bias[inter + i]; }
        ie_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 in and out, width a multiple of 8: a thread takes eight gates and their ups as two 16-byte
// loads, the row from the grid (no division); biases, activation in 32-bit (precise exponential and divide).
__global__ void __launch_bounds__(256)
silu_mul_bias_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, const float* __restrict__ bias,
                            __nv_bfloat16* __restrict__ out, int inter) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t row = blockIdx.y;
    int v = blockIdx.x * 256 + threadIdx.x;
    if (v >= inter / 8) return;
    const __nv_bfloat16* g_row = gate_up + row * 2 * inter;
    uint4 graw = *reinterpret_cast<const uint4*>(g_row + v * 8);
    uint4 uraw = *reinterpret_cast<const uint4*>(g_row + inter + v * 8);
    float bg[8], bu[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        bg[j] = bias ? bias[v * 8 + j] : 0.f;
        bu[j] = bias ? bias[inter + v * 8 + j] : 0.f;
    }
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 gf = __bfloat1622float2(g2[j]), uf = __bfloat1622float2(u2[j]);
        float g0 = gf.x + bg[2 * j], g1 = gf.y + bg[2 * j + 1];
        float u0 = uf.x + bu[2 * j], u1 = uf.y + bu[2 * j + 1];
        o2[j] = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
    }
    *reinterpret_cast<uint4*>(out + row * inter + (size_t)v * 8) = oraw;
}

template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out,
                                   int width, size_t total) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        size_t row = idx / (2 * width);
        int i = (int)(idx - row * 2 * width);
        float v = i < width ? a[row * width + i] : b[row * width + (i - width)];
        ie_store(out + idx, v);
    }
}

__global__ void weighted_sum_kernel(const float* __restrict__ a, float sa, const float* __restrict__ b, float sb,
                                    float* __restrict__ out, size_t total) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) out[idx] = fmaf(sb, b[idx], sa * a[idx]);
}

inline int grid_for(size_t total, int threads) {
    size_t want = (total + threads - 1) / threads;
    return (int)(want < 148 * 16 ? want : 148 * 16);
}
}  // namespace

IE_API int ie_bigram_embedding(const void* embed, const void* bigram, int table_dtype, const int* ids,
                               const int* positions, const int* seq_of_token, const int* cu_q, const int* slots,
                               void* state, long long state_stride, int num_slots, float* out, int num_tokens,
                               int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur, int* err,
                               void* stream) {
    if (num_tokens <= 0) return 0;
    if (buckets < 1) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == IE_BF16)
        return ie_launch(bigram_embedding_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, s,
                         (const __nv_bfloat16*)embed, (const __nv_bfloat16*)bigram, ids, positions, seq_of_token, cu_q,
                         slots, (int*)state, state_stride, num_slots, out, hidden, vocab, buckets, mul_prev, mul_cur, err);
    return ie_launch(bigram_embedding_kernel<float>, dim3(num_tokens), dim3(128), 0, s, (const float*)embed,
                     (const float*)bigram, ids, positions, seq_of_token, cu_q, slots, (int*)state, state_stride,
                     num_slots, out, hidden, vocab, buckets, mul_prev, mul_cur, err);
}

// `out` may be null (only the residual stream is brought up to date); `delta` may be null (a plain
// norm of h); `rows` selects rows, and then h is not modified.
IE_API int ie_sandwich_norm(float* h, const float* delta, int num_partials, long long partial_stride,
                            const float* delta2, int num_partials2, long long partial_stride2,
                            const float* extra, const float* bias, const float* post_w, float post_eps, const float* pre_w,
                            float pre_eps, void* out, int out_dtype, const int* rows, int num_rows, int hidden,
                            void* stream) {
    if (num_rows <= 0) return 0;
    if (delta != nullptr && num_partials < 1) return (int)cudaErrorInvalidValue;
    if (delta == nullptr && (delta2 != nullptr || extra != nullptr)) return (int)cudaErrorInvalidValue;
    if (delta2 == nullptr) num_partials2 = 0;
    if (out != nullptr && pre_w == nullptr) return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    bool vec = hidden % 4 == 0 && (size_t)partial_stride % 4 == 0 && (size_t)partial_stride2 % 4 == 0 &&
               ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(bias) |
                 reinterpret_cast<uintptr_t>(delta2) | reinterpret_cast<uintptr_t>(extra) |
                 reinterpret_cast<uintptr_t>(post_w) | reinterpret_cast<uintptr_t>(pre_w) |
                 reinterpret_cast<uintptr_t>(out)) % 16 == 0);
#define IE_SN_LAUNCH(T, V)                                                                                         \
    do {                                                                                                           \
        static IePerDevice allowed;                                                                                \
        if (smem > 48 * 1024) {                                                                                    \
            cudaError_t e = ie_allow_smem(allowed, sandwich_norm_kernel<T, V>, 200 * 1024);                        \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return ie_launch(sandwich_norm_kernel<T, V>, dim3(num_rows), dim3(SN_THREADS), smem, s, h, delta,          \
                         num_partials, (size_t)partial_stride, delta2, num_partials2, (size_t)partial_stride2,     \
                         extra, bias, post_w, post_eps, pre_w, pre_eps, (T*)out, rows, hidden);                    \
    } while (0)
    if (out_dtype == IE_BF16) {
        if (vec) IE_SN_LAUNCH(__nv_bfloat16, 4);
        IE_SN_LAUNCH(__nv_bfloat16, 1);
    }
    if (vec) IE_SN_LAUNCH(float, 4);
    IE_SN_LAUNCH(float, 1);
#undef IE_SN_LAUNCH
}

// `gate_up` is 32-bit, or has the output's dtype (the product's sums rounded once before the biases).
IE_API int ie_silu_mul_bias(const void* gate_up, int in_dtype, const float* bias, void* out, int out_dtype,
                            int num_rows, int inter, void* stream) {
    size_t total = (size_t)num_rows * inter;
    if (total == 0) return 0;
    if (in_dtype != IE_F32 && in_dtype != out_dtype) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16 && in_dtype == IE_BF16 && inter % 8 == 0 && num_rows <= 65535)
        return ie_launch(silu_mul_bias_bf16x8_kernel, dim3((unsigned)((inter / 8 + 255) / 256), (unsigned)num_rows),
                         dim3(256), 0, s, (const __nv_bfloat16*)gate_up, bias, (__nv_bfloat16*)out, inter);
    if (out_dtype == IE_BF16 && in_dtype == IE_BF16)
        return ie_launch(silu_mul_bias_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid_for(total, 256)), dim3(256), 0,
                         s, (const __nv_bfloat16*)gate_up, bias, (__nv_bfloat16*)out, inter, total);
    if (out_dtype == IE_BF16)
        return ie_launch(silu_mul_bias_kernel<__nv_bfloat16, float>, dim3(grid_for(total, 256)), dim3(256), 0, s,
                         (const float*)gate_up, bias, (__nv_bfloat16*)out, inter, total);
    return ie_launch(silu_mul_bias_kernel<float, float>, dim3(grid_for(total, 256)), dim3(256), 0, s,
                     (const float*)gate_up, bias, (float*)out, inter, total);
}

IE_API int ie_concat_cast(const float* a, const float* b, void* out, int out_dtype, int num_rows, int width,
                          void* stream) {
    size_t total = (size_t)num_rows * 2 * width;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16)
        return ie_launch(concat_cast_kernel<__nv_bfloat16>, dim3(grid_for(total, 256)), dim3(256), 0, s, a, b,
                         (__nv_bfloat16*)out, width, total);
    return ie_launch(concat_cast_kernel<float>, dim3(grid_for(total, 256)), dim3(256), 0, s, a, b, (float*)out, width,
                     total);
}

IE_API int ie_weighted_sum(const float* a, float sa, const float* b, float sb, float* out, long long total,
                           void* stream) {
    if (total <= 0) return 0;
    return ie_launch(weighted_sum_kernel, dim3(grid_for((size_t)total, 256)), dim3(256), 0, (cudaStream_t)stream, a,
                     sa, b, sb, out, (size_t)total);
}

// `delta` is the sum of `num_partials` arrays; `out` may be null (only h is brought up to date);
// `rows` selects rows, and then h is not modified.
IE_API int ie_gated_add_norm(float* h, const float* delta, int num_partials, long long partial_stride,
                             const float* gate_pre, int gate_partials, long long gate_stride, int gate_ld,
                             const float* gate_bias, const float* weight, float eps,
                             void* out, int out_dtype, const int* rows, int num_rows, int hidden, void* stream) {
    if (num_rows <= 0) return 0;
    if (delta == nullptr || gate_pre == nullptr || num_partials < 1 || gate_partials < 1 || gate_ld < hidden)
        return (int)cudaErrorInvalidValue;
    if (out != nullptr && weight == nullptr) return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    bool vec = hidden % 4 == 0 && (size_t)partial_stride % 4 == 0 && (size_t)gate_stride % 4 == 0 && gate_ld % 4 == 0 &&
               ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(delta) |
                 reinterpret_cast<uintptr_t>(gate_pre) | reinterpret_cast<uintptr_t>(gate_bias) |
                 reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) % 16 == 0);
#define IE_GN_LAUNCH(T, V)                                                                                         \
    do {                                                                                                           \
        static IePerDevice allowed;                                                                                \
        if (smem > 48 * 1024) {                                                                                    \
            cudaError_t e = ie_allow_smem(allowed, gated_add_norm_kernel<T, V>, 200 * 1024);                       \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return ie_launch(gated_add_norm_kernel<T, V>, dim3(num_rows), dim3(SN_THREADS), smem, s, h, delta,         \
                         num_partials, (size_t)partial_stride, gate_pre, gate_partials, (size_t)gate_stride,       \
                         gate_ld, gate_bias, weight, eps, (T*)out, rows, hidden);                                  \
    } while (0)
    if (out_dtype == IE_BF16) {
        if (vec) IE_GN_LAUNCH(__nv_bfloat16, 4);
        IE_GN_LAUNCH(__nv_bfloat16, 1);
    }
    if (vec) IE_GN_LAUNCH(float, 4);
    IE_GN_LAUNCH(float, 1);
#undef IE_GN_LAUNCH
}

// `z` is 32-bit or has the output's dtype.
IE_API int ie_polynorm(const void* z, int z_ld, int in_dtype, const float* coeff, float eps, void* out,
                       int out_dtype, int num_rows, int width, void* stream) {
    if (num_rows <= 0 || width <= 0) return 0;
    if (z_ld < width) return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024 || (in_dtype != IE_F32 && in_dtype != out_dtype)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
#define IE_PN_LAUNCH(IN, OUT)                                                                                      \
    do {                                                                                                           \
        static IePerDevice allowed;                                                                                \
        if (smem > 48 * 1024) {                                                                                    \
            cudaError_t e = ie_allow_smem(allowed, polynorm_kernel<IN, OUT>, 200 * 1024);                          \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return ie_launch(polynorm_kernel<IN, OUT>, dim3(num_rows), dim3(SN_THREADS), smem, s, (const IN*)z, z_ld,   \
                         coeff, eps, (OUT*)out, width);                                                            \
    } while (0)
    if (out_dtype == IE_BF16) {
        if (in_dtype == IE_BF16) IE_PN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
        IE_PN_LAUNCH(float, __nv_bfloat16);
    }
    IE_PN_LAUNCH(float, float);
#undef IE_PN_LAUNCH
}
