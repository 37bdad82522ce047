// Input stage of an attention whose queries and keys are normalised per head before the rotation,
// and whose value rows may have another size than its key rows.  Variants by parameters: a bias on
// the whole projection (`bias`, laid out like a row of it, added first); no norm on queries or keys
// (their weight is null); value heads divided by their root mean square over `vdim` (eps inside the
// root, no weight) before they are cached (`value_norm`); values that are the keys as projected
// (with their bias, before norm and rotation: `values_from_keys`; the projection then holds no value
// columns and vdim = dim); the rotation's pairs (`interleaved` 0: entry i with entry i + rot_dims / 2;
// 1: entry 2i with entry 2i + 1; the table of angles is the same).
//
// qk_norm_rope_write: from the fused 32-bit projection [N, ld] = (heads * dim queries, kv_heads *
// dim keys, kv_heads * vdim values): every query and key head is divided by its root mean square
// over `dim` (eps inside the root) and multiplied by a weight of size `dim` that all heads share;
// the first rot_dims entries of the head are rotated by the token's position (entry i pairs with
// entry i + rot_dims / 2; cos and sin come from the 32-bit table [positions, 2, rot_dims / 2]);
// queries go to q_out [N, heads * dim], keys and values into the request's page rows
// (k_cache [pages, kv_heads, page_size, dim], v_cache [pages, kv_heads, page_size, vdim]).
// One warp per (token, head of q, k or v); the sums do not depend on the rest of the step.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int QW_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(QW_WARPS * 32)
qk_norm_rope_write_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ positions,
                          const float* __restrict__ table, int rot_dims, int table_positions,
                          const float* __restrict__ bias, int value_norm, int values_from_keys, int interleaved,
                          const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                          T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                          const int* __restrict__ slot_mapping, int heads, int kv_heads, int dim, int vdim,
                          int page_size, int total_pages, int* err) {
    extern __shared__ float rows[];  // [QW_WARPS][dim]
    ie_pdl_trigger();
    ie_pdl_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int unit = blockIdx.y * QW_WARPS + warp;
    int n = blockIdx.x;
    int units = heads + 2 * kv_heads;
    if (unit >= units) return;
    const float* src = proj + (size_t)n * ld;
    long long cache_row = -1;
    if (unit >= heads) {
        if (slot_mapping == nullptr) return;  // a run that borrows another layer's cache writes nothing
        int slot = slot_mapping[n];
        int page = slot / page_size;
        if (slot < 0 || page >= total_pages) {
            if (lane == 0) ie_report(err, IE_ERR_PAGE, slot, n);
            return;
        }
        int g = (unit - heads) % kv_heads;
        cache_row = ((long long)page * kv_heads + g) * page_size + (slot % page_size);
    }
    if (unit >= heads + kv_heads) {  // a value head: copied as it is, or divided by its root mean square
        int g = unit - heads - kv_heads;
        size_t col = values_from_keys ? (size_t)(heads + g) * dim : (size_t)(heads + kv_heads) * dim + (size_t)g * vdim;
        const float* v = src + col;
        const float* vb = bias != nullptr ? bias + col : nullptr;
        float inv = 1.0f;
        if (value_norm) {
            float ss = 0.f;
            for (int d = lane; d < vdim; d += 32) {
                float e = vb != nullptr ? v[d] + vb[d] : v[d];
                ss = fmaf(e, e, ss);
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)vdim + eps);
        }
        for (int d = lane; d < vdim; d += 32)
            ie_store(v_cache + cache_row * vdim + d, (vb != nullptr ? v[d] + vb[d] : v[d]) * inv);
        return;
    }
    bool is_q = unit < heads;
    const float* x = src + (size_t)unit * dim;  // (the key heads follow the query heads)
    const float* xb = bias != nullptr ? bias + (size_t)unit * dim : nullptr;
    const float* weight = is_q ? q_weight : k_weight;
    float* y = rows + warp * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) {
        float e = xb != nullptr ? x[d] + xb[d] : x[d];
        y[d] = e;
        ss = fmaf(e, e, ss);
    }
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    if (weight != nullptr)
        for (int d = lane; d < dim; d += 32) y[d] = (y[d] * inv) * weight[d];
    __syncwarp();
    int pos = positions[n];
    int half = rot_dims / 2;
    if (half > 0 && (pos < 0 || pos >= table_positions)) {
        if (lane == 0) ie_report(err, IE_ERR_POSITION, pos, n);
        return;
    }
    T* dst = is_q ? q_out + ((size_t)n * heads + unit) * dim : k_cache + cache_row * dim;
    for (int d = lane; d < dim; d += 32) {
        float r = y[d];
        if (interleaved) {
            if (d < rot_dims) {
                int j = d >> 1;
                float c = table[((size_t)pos * 2) * half + j], s = table[((size_t)pos * 2 + 1) * half + j];
                r = (d & 1) ? y[d] * c + y[d - 1] * s : y[d] * c - y[d + 1] * s;
            }
        } else if (d < half) {
            float c = table[((size_t)pos * 2) * half + d], s = table[((size_t)pos * 2 + 1) * half + d];
            r = y[d] * c - y[d + half] * s;
        } else if (d < rot_dims) {
            float c = table[((size_t)pos * 2) * half + (d - half)], s = table[((size_t)pos * 2 + 1) * half + (d - half)];
            r = y[d] * c + y[d - half] * s;
        }
        ie_store(dst + d, r);
    }
}
}  // namespace

IE_API int ie_qk_norm_rope_write(const float* proj, int ld, const int* positions, const float* table, int rot_dims,
                                 int table_positions, const float* bias, int value_norm, int values_from_keys,
                                 int interleaved, const float* q_weight,
                                 const float* k_weight, float eps,
                                 void* q_out, void* k_cache, void* v_cache, int dtype, const int* slot_mapping,
                                 int num_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                                 int total_pages, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dim || (rot_dims > 0 && table == nullptr))
        return (int)cudaErrorInvalidValue;
    if (values_from_keys && vdim != dim) return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)QW_WARPS * dim * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    int units = heads + 2 * kv_heads;
    dim3 grid(num_tokens, (units + QW_WARPS - 1) / QW_WARPS);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        return ie_launch(qk_norm_rope_write_kernel<__nv_bfloat16>, grid, dim3(QW_WARPS * 32), smem, s, proj, ld,
                         positions, table, rot_dims, table_positions, bias, value_norm, values_from_keys, interleaved, q_weight, k_weight, eps, (__nv_bfloat16*)q_out,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping, heads, kv_heads, dim, vdim,
                         page_size, total_pages, err);
    return ie_launch(qk_norm_rope_write_kernel<float>, grid, dim3(QW_WARPS * 32), smem, s, proj, ld, positions, table,
                     rot_dims, table_positions, bias, value_norm, values_from_keys, interleaved, q_weight, k_weight, eps, (float*)q_out, (float*)k_cache,
                     (float*)v_cache, slot_mapping, heads, kv_heads, dim, vdim, page_size, total_pages, err);
}
