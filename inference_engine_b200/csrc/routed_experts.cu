// Kernels of the routed feed-forward (many small gated experts, a few per token).
//
//  * route_topk: per token the router's logits (32-bit; plus a bias per expert if the router has
//    one), their softmax over all experts, the
//    groups' best scores, the kept groups, the `top` best allowed experts (ties: the lower index)
//    and their scores divided by their sum (+ 1e-20), times `weight_scale`.  With `sigmoid_scores` an
//    expert's score is the sigmoid of its logit instead; a `correction` per expert is then added for
//    the choice alone (groups and experts are chosen by score + correction, the weights are the plain
//    scores), a group is ranked by its best `group_top` (1 or 2) corrected scores added up, and the
//    experts of groups that are not kept cannot be chosen whatever their sign.
//  * routed_align: the step's (token, choice) pairs sorted by expert into tiles of TILE_M rows:
//    every expert's run of pairs is padded to whole tiles (padding rows are -1), and a list says
//    which expert each tile belongs to.  One block; nothing goes to the host.
//  * routed_gate_up: per tile and 64 columns: gate and up products of the tile's tokens with the
//    tile's expert, then  g = min(gate, limit), u = clamp(up, -limit, limit),
//    y = g * sigmoid(alpha * g) * (u + up_offset), written per pair.
//  * routed_down: per tile and 64 columns: y times the expert's down matrix, times the pair's
//    routing weight, written to out[choice][token][:]; the consumer adds the `top` slices in order.
// bfloat16 products run on mma.sync.m16n8k16 with 32-bit sums, 32-bit products on fused
// multiply-adds; a row's sums run over k in a fixed order, whatever else is in the tile.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int ROUTE_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_topk_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, int width,
                  int experts, int top, int groups, int keep, int sigmoid_scores,
                  const float* __restrict__ correction, int group_top, float weight_scale,
                  int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float sm[];  // x[width], score[experts], group_best[groups], choice[experts]
    float* xs = sm;
    float* score = xs + width;
    float* gbest = score + experts;
    float* choice = gbest + groups;
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < width; i += ROUTE_THREADS) xs[i] = ie_load(x + (size_t)n * width + i);
    __syncthreads();
    // A warp takes the experts warp, warp + 8, ...; four of them at a time, so that four rows' loads are
    // on their way together.  An expert's sum is the same chain of operations whichever way it is grouped.
    constexpr int WARPS = ROUTE_THREADS / 32, AT_ONCE = 4;
    for (int e0 = warp; e0 < experts; e0 += WARPS * AT_ONCE) {
        float acc[AT_ONCE];
        if (width % 4 == 0) {  // (four partial sums per lane and expert, added in a fixed order)
            float a4[AT_ONCE][4];
#pragma unroll
            for (int u = 0; u < AT_ONCE; ++u) a4[u][0] = a4[u][1] = a4[u][2] = a4[u][3] = 0.f;
            for (int i = lane * 4; i < width; i += 128) {
                float4 xv = *reinterpret_cast<const float4*>(xs + i);
#pragma unroll
                for (int u = 0; u < AT_ONCE; ++u) {
                    int e = e0 + u * WARPS;
                    if (e < experts) {
                        float4 wv = *reinterpret_cast<const float4*>(w + (size_t)e * width + i);
                        a4[u][0] = fmaf(xv.x, wv.x, a4[u][0]); a4[u][1] = fmaf(xv.y, wv.y, a4[u][1]);
                        a4[u][2] = fmaf(xv.z, wv.z, a4[u][2]); a4[u][3] = fmaf(xv.w, wv.w, a4[u][3]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < AT_ONCE; ++u) acc[u] = (a4[u][0] + a4[u][1]) + (a4[u][2] + a4[u][3]);
        } else {
#pragma unroll
            for (int u = 0; u < AT_ONCE; ++u) {
                int e = e0 + u * WARPS;
                acc[u] = 0.f;
                if (e < experts)
                    for (int i = lane; i < width; i += 32) acc[u] = fmaf(xs[i], w[(size_t)e * width + i], acc[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u) {
            int e = e0 + u * WARPS;
            float total = warp_sum(acc[u]);
            if (lane == 0 && e < experts) score[e] = bias != nullptr ? total + bias[e] : total;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (sigmoid_scores) {
        for (int e = lane; e < experts; e += 32) {
            float sg = 1.0f / (1.0f + expf(-score[e]));
            score[e] = sg;
            choice[e] = correction != nullptr ? sg + correction[e] : sg;
        }
        __syncwarp();
        int per = experts / groups;
        if (keep < groups) {
            for (int g = lane; g < groups; g += 32) {  // the group's best corrected scores, one or two of them
                float b1 = -INFINITY, b2 = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    float c = choice[e];
                    if (c > b1) { b2 = b1; b1 = c; }
                    else if (c > b2) b2 = c;
                }
                gbest[g] = (group_top >= 2 && per >= 2) ? b1 + b2 : b1;
            }
        }
        __syncwarp();
        if (lane != 0) return;
        if (keep < groups) {
            for (int round = 0; round < keep; ++round) {  // (a kept group is marked by +inf; ties: the lower index)
                int best = -1;
                float bv = -INFINITY;
                for (int g = 0; g < groups; ++g)
                    if (gbest[g] != INFINITY && (best < 0 || gbest[g] > bv)) { bv = gbest[g]; best = g; }
                if (best < 0) break;
                gbest[best] = INFINITY;
            }
            for (int g = 0; g < groups; ++g)
                if (gbest[g] != INFINITY)
                    for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
        }
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (choice[e] > bv) { bv = choice[e]; best = e; }
            float wj = best < 0 ? 0.f : score[best];
            ids[(size_t)n * top + j] = best < 0 ? 0 : best;
            weights[(size_t)n * top + j] = wj;
            total += wj;
            if (best >= 0) choice[best] = -INFINITY;  // taken
        }
        float f = weight_scale / (total + 1e-20f);
        for (int j = 0; j < top; ++j) weights[(size_t)n * top + j] *= f;
        return;
    }
    // softmax over all experts (lanes share the work, every lane ends with the same numbers)
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, score[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
        float p = expf(score[e] - m);
        score[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    float inv = 1.0f / sum;
    for (int e = lane; e < experts; e += 32) score[e] *= inv;
    __syncwarp();
    int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
        float b = -1.f;
        for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, score[e]);
        gbest[g] = b;
    }
    __syncwarp();
    if (lane != 0) return;
    // keep the best groups: a group that is not kept gets its experts' scores hidden (negated - 1)
    if (keep < groups) {
        for (int round = 0; round < keep; ++round) {
            int best = -1;
            float bv = -1.f;
            for (int g = 0; g < groups; ++g)
                if (gbest[g] >= 0.f && gbest[g] > bv) { bv = gbest[g]; best = g; }
            if (best < 0) break;
            gbest[best] = -2.f - gbest[best];  // marked as kept
        }
        for (int g = 0; g < groups; ++g)
            if (gbest[g] >= 0.f)
                for (int e = g * per; e < (g + 1) * per; ++e) score[e] = -1.f - score[e];
    }
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        int best = 0;
        float bv = -1.f;
        for (int e = 0; e < experts; ++e)
            if (score[e] >= 0.f && score[e] > bv) { bv = score[e]; best = e; }
        ids[(size_t)n * top + j] = best;
        weights[(size_t)n * top + j] = bv < 0.f ? 0.f : bv;
        total += bv < 0.f ? 0.f : bv;
        score[best] = -1.f - score[best];  // taken
    }
    float f = weight_scale / (total + 1e-20f);
    for (int j = 0; j < top; ++j) weights[(size_t)n * top + j] *= f;
}

constexpr int TILE_M = 64, TILE_N = 64, TILE_K = 32;

// sorted[tiles * TILE_M]: pair index (token * top + choice) or -1; tile_expert[tiles]; meta[0] = tiles.
__global__ void __launch_bounds__(1024)
routed_align_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ sorted,
                    int* __restrict__ tile_expert, int* __restrict__ meta, int max_tiles) {
    extern __shared__ int ism[];  // count[experts], first[experts] (first row of the expert's run), cursor[experts]
    int* count = ism;
    int* first = count + experts;
    int* cursor = first + experts;
    ie_pdl_trigger();
    ie_pdl_wait();
    int tid = threadIdx.x;
    for (int e = tid; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    for (int i = tid; i < max_tiles * TILE_M; i += blockDim.x) sorted[i] = -1;
    __syncthreads();
    for (int i = tid; i < pairs; i += blockDim.x) {
        int e = ids[i];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int tiles = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = tiles * TILE_M;
            int t = (count[e] + TILE_M - 1) / TILE_M;
            for (int j = 0; j < t && tiles + j < max_tiles; ++j) tile_expert[tiles + j] = e;
            tiles += t;
        }
        meta[0] = tiles < max_tiles ? tiles : max_tiles;
    }
    __syncthreads();
    for (int i = tid; i < pairs; i += blockDim.x) {
        int e = ids[i];
        if (e < 0 || e >= experts) continue;
        int at = first[e] + atomicAdd(&cursor[e], 1);
        if (at < max_tiles * TILE_M) sorted[at] = i;
    }
}

// ---- tile products -----------------------------------------------------------------------------
// A tile: up to TILE_M rows (given by pointers, nullptr = a padding row of zeros) times TILE_N rows
// of a [*, K] matrix, over all of K.  128 threads.

// 32-bit: thread (ty, tx) of 8 x 16 owns rows ty*8 .. +7 and columns tx*4 .. +3.
struct TileF32 {
    static constexpr int ACC = 32;
    float (*as)[TILE_M + 4];
    float (*bs)[TILE_N + 4];
    __device__ void zero(float* acc) {
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    }
    __device__ void load_a(const float* const* rows, int k0, int K) {
        for (int i = threadIdx.x; i < TILE_M * TILE_K; i += 128) {
            int r = i / TILE_K, k = i - r * TILE_K;
            const float* p = rows[r];
            as[k][r] = (p != nullptr && k0 + k < K) ? p[k0 + k] : 0.f;
        }
    }
    __device__ void load_b(const float* w, int n0, int N, int k0, int K) {
        for (int i = threadIdx.x; i < TILE_N * TILE_K; i += 128) {
            int r = i / TILE_K, k = i - r * TILE_K;
            bs[k][r] = (n0 + r < N && k0 + k < K) ? w[(size_t)(n0 + r) * K + k0 + k] : 0.f;
        }
    }
    __device__ void mma(float* acc) {
        int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
        for (int k = 0; k < TILE_K; ++k) {
            float a[8], b[4];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = as[k][ty * 8 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i * 4 + j] = fmaf(a[i], b[j], acc[i * 4 + j]);
        }
    }
    // element e of a thread's accumulators -> (row, column) inside the tile
    __device__ static void where(int e, int& r, int& c) {
        r = (threadIdx.x >> 4) * 8 + e / 4;
        c = (threadIdx.x & 15) * 4 + e % 4;
    }
};

// bfloat16: warp w of 4 owns rows (w >> 1) * 32 .. +31 and columns (w & 1) * 32 .. +31: two 16-row
// and four 8-column instruction tiles.
struct TileBF16 {
    static constexpr int ACC = 32;
    static constexpr int LD = TILE_K + 8;  // bfloat16 per shared-memory row (80 bytes: no bank conflicts)
    __nv_bfloat16 (*as)[LD];
    __nv_bfloat16 (*bs)[LD];
    __device__ void zero(float* acc) {
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    }
    __device__ static void load_rows(__nv_bfloat16 (*dst)[LD], int r, int seg, const __nv_bfloat16* p, int k0, int K, bool vec) {
        // 8 entries (16 bytes) of row r from column k0 + seg * 8
        int k = k0 + seg * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (p != nullptr) {
            if (vec && k + 8 <= K) v = *reinterpret_cast<const uint4*>(p + k);
            else {
                __nv_bfloat16 tmp[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) tmp[i] = (k + i < K) ? p[k + i] : __float2bfloat16_rn(0.f);
                v = *reinterpret_cast<uint4*>(tmp);
            }
        }
        *reinterpret_cast<uint4*>(&dst[r][seg * 8]) = v;
    }
    __device__ void load_a(const __nv_bfloat16* const* rows, int k0, int K) {
        bool vec = (K % 8 == 0);
        for (int i = threadIdx.x; i < TILE_M * (TILE_K / 8); i += 128) {
            int r = i >> 2, seg = i & 3;
            load_rows(as, r, seg, rows[r], k0, K, vec);
        }
    }
    __device__ void load_b(const __nv_bfloat16* w, int n0, int N, int k0, int K) {
        bool vec = (K % 8 == 0);
        for (int i = threadIdx.x; i < TILE_N * (TILE_K / 8); i += 128) {
            int r = i >> 2, seg = i & 3;
            load_rows(bs, r, seg, n0 + r < N ? w + (size_t)(n0 + r) * K : nullptr, k0, K, vec);
        }
    }
    __device__ void mma(float* acc) {
        int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        int rm = (warp >> 1) * 32, cn = (warp & 1) * 32;
#pragma unroll
        for (int kk = 0; kk < TILE_K; kk += 16) {
            unsigned a[2][4], b[4][2];
            // A: a 16 x 16 tile per x4; B: two 8-column tiles (both halves of k) per x4
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                unsigned addr = (unsigned)__cvta_generic_to_shared(&as[rm + mi * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a[mi][0]), "=r"(a[mi][1]), "=r"(a[mi][2]), "=r"(a[mi][3]) : "r"(addr));
            }
#pragma unroll
            for (int nj = 0; nj < 4; nj += 2) {
                unsigned addr = (unsigned)__cvta_generic_to_shared(
                    &bs[cn + nj * 8 + (lane & 7) + ((lane >> 4) & 1) * 8][kk + ((lane >> 3) & 1) * 8]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b[nj][0]), "=r"(b[nj][1]), "=r"(b[nj + 1][0]), "=r"(b[nj + 1][1]) : "r"(addr));
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    float* c = acc + (mi * 4 + ni) * 4;
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                        : "r"(a[mi][0]), "r"(a[mi][1]), "r"(a[mi][2]), "r"(a[mi][3]), "r"(b[ni][0]), "r"(b[ni][1]));
                }
        }
    }
    __device__ static void where(int e, int& r, int& c) {
        int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        int mi = e / 16, ni = (e / 4) % 4, j = e % 4;
        r = (warp >> 1) * 32 + mi * 16 + (lane >> 2) + (j >> 1) * 8;
        c = (warp & 1) * 32 + ni * 8 + (lane & 3) * 2 + (j & 1);
    }
};

template <typename T> struct TileOf;
template <> struct TileOf<float> { using type = TileF32; };
template <> struct TileOf<__nv_bfloat16> { using type = TileBF16; };

template <typename T>
__device__ __forceinline__ typename TileOf<T>::type make_tile(unsigned char* raw) {
    typename TileOf<T>::type tile;
    if constexpr (sizeof(T) == 4) {
        tile.as = reinterpret_cast<float (*)[TILE_M + 4]>(raw);
        tile.bs = reinterpret_cast<float (*)[TILE_N + 4]>(raw + sizeof(float) * TILE_K * (TILE_M + 4));
    } else {
        tile.as = reinterpret_cast<__nv_bfloat16 (*)[TileBF16::LD]>(raw);
        tile.bs = reinterpret_cast<__nv_bfloat16 (*)[TileBF16::LD]>(raw + sizeof(__nv_bfloat16) * TILE_M * TileBF16::LD);
    }
    return tile;
}

constexpr size_t TILE_SMEM_F32 = sizeof(float) * TILE_K * (TILE_M + 4 + TILE_N + 4);
constexpr size_t TILE_SMEM = TILE_SMEM_F32;  // the bfloat16 tiles need less

// x: [N, K]; w_gate_up: [experts, 2, F, K]; y: [pairs, F].
template <typename T>
__global__ void __launch_bounds__(128)
routed_gate_up_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                      const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                      const int* __restrict__ meta, int top, int K, int F, float limit, int clamp,
                      float alpha, float up_offset) {
    __shared__ __align__(16) unsigned char raw[TILE_SMEM];
    __shared__ const T* rows[TILE_M];
    __shared__ int pair_of[TILE_M];
    ie_pdl_trigger();
    ie_pdl_wait();
    int tile_id = blockIdx.y;
    if (tile_id >= meta[0]) return;
    int e = tile_expert[tile_id], n0 = blockIdx.x * TILE_N;
    if (threadIdx.x < TILE_M) {
        int pair = sorted[tile_id * TILE_M + threadIdx.x];
        pair_of[threadIdx.x] = pair;
        rows[threadIdx.x] = pair >= 0 ? x + (size_t)(pair / top) * K : nullptr;
    }
    __syncthreads();
    auto tile = make_tile<T>(raw);
    const T* wg = w + (size_t)e * 2 * F * K;
    const T* wu = wg + (size_t)F * K;
    float gate[32], up[32];
    tile.zero(gate);
    tile.zero(up);
    for (int k0 = 0; k0 < K; k0 += TILE_K) {
        tile.load_a(rows, k0, K);
        tile.load_b(wg, n0, F, k0, K);
        __syncthreads();
        tile.mma(gate);
        __syncthreads();
        tile.load_b(wu, n0, F, k0, K);
        __syncthreads();
        tile.mma(up);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        int r, c;
        tile.where(i, r, c);
        int pair = pair_of[r];
        if (pair < 0 || n0 + c >= F) continue;
        float g = gate[i], u = up[i];
        if (clamp) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        float act = g / (1.0f + expf(-alpha * g)) * (u + up_offset);
        ie_store(y + (size_t)pair * F + n0 + c, act);
    }
}

// y: [pairs, F]; w_down: [experts, H, F]; out: [top, N, H] 32-bit.
template <typename T>
__global__ void __launch_bounds__(128)
routed_down_kernel(const T* __restrict__ y, const T* __restrict__ w, float* __restrict__ out,
                   const float* __restrict__ weights, const int* __restrict__ sorted,
                   const int* __restrict__ tile_expert, const int* __restrict__ meta, int top, int N,
                   int F, int H) {
    __shared__ __align__(16) unsigned char raw[TILE_SMEM];
    __shared__ const T* rows[TILE_M];
    __shared__ int pair_of[TILE_M];
    ie_pdl_trigger();
    ie_pdl_wait();
    int tile_id = blockIdx.y;
    if (tile_id >= meta[0]) return;
    int e = tile_expert[tile_id], n0 = blockIdx.x * TILE_N;
    if (threadIdx.x < TILE_M) {
        int pair = sorted[tile_id * TILE_M + threadIdx.x];
        pair_of[threadIdx.x] = pair;
        rows[threadIdx.x] = pair >= 0 ? y + (size_t)pair * F : nullptr;
    }
    __syncthreads();
    auto tile = make_tile<T>(raw);
    const T* wd = w + (size_t)e * H * F;
    float acc[32];
    tile.zero(acc);
    for (int k0 = 0; k0 < F; k0 += TILE_K) {
        tile.load_a(rows, k0, F);
        tile.load_b(wd, n0, H, k0, F);
        __syncthreads();
        tile.mma(acc);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        int r, c;
        tile.where(i, r, c);
        int pair = pair_of[r];
        if (pair < 0 || n0 + c >= H) continue;
        int token = pair / top, choice = pair - token * top;
        out[((size_t)choice * N + token) * H + n0 + c] = weights[pair] * acc[i];
    }
}

// ---- bfloat16 with rows that are multiples of 16 bytes: the same tiles fed by cp.async -------------
// Three stages of (rows of A, NB matrices' rows) in flight; one barrier per 32 columns of k.
// NB = 2: gate and up, then the activation; NB = 1: the down product, times the routing weight.
constexpr int PIPE_STAGES = 3;
constexpr int PIPE_LD = TileBF16::LD;
constexpr size_t pipe_smem(int nb) { return (size_t)PIPE_STAGES * (1 + nb) * TILE_M * PIPE_LD * sizeof(__nv_bfloat16); }

__device__ __forceinline__ void cp16(void* dst, const void* src, int bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int NB>
__global__ void __launch_bounds__(128)
routed_bf16_kernel(const __nv_bfloat16* __restrict__ a_rows, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ out, const float* __restrict__ weights,
                   const int* __restrict__ sorted, const int* __restrict__ tile_expert, const int* __restrict__ meta,
                   int top, int N, int K, int F, float limit, int clamp, float alpha, float up_offset) {
    // NB = 2: a_rows = x [N, K], w = [experts, 2, F, K], output y [pairs, F]
    // NB = 1: a_rows = y [pairs, K], w = [experts, F, K] (F = the model's width), output out [top, N, F]
    extern __shared__ __align__(16) unsigned char pipe_raw[];
    __shared__ const __nv_bfloat16* rows[TILE_M];
    __shared__ int pair_of[TILE_M];
    ie_pdl_trigger();
    ie_pdl_wait();
    int tile_id = blockIdx.y;
    if (tile_id >= meta[0]) return;
    int e = tile_expert[tile_id], n0 = blockIdx.x * TILE_N;
    if (threadIdx.x < TILE_M) {
        int pair = sorted[tile_id * TILE_M + threadIdx.x];
        pair_of[threadIdx.x] = pair;
        rows[threadIdx.x] = pair < 0 ? nullptr : a_rows + (size_t)(NB == 2 ? pair / top : pair) * K;
    }
    __syncthreads();
    auto stage_ptr = [&](int stage, int which) {
        return reinterpret_cast<__nv_bfloat16(*)[PIPE_LD]>(
            pipe_raw + ((size_t)stage * (1 + NB) + which) * TILE_M * PIPE_LD * sizeof(__nv_bfloat16));
    };
    const __nv_bfloat16* wb[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) wb[b] = w + ((size_t)e * NB + b) * F * K;
    auto issue = [&](int it) {
        int stage = it % PIPE_STAGES, k0 = it * TILE_K;
        for (int i = threadIdx.x; i < TILE_M * (TILE_K / 8); i += 128) {
            int r = i >> 2, k = k0 + (i & 3) * 8;
            bool in_k = k < K;
            const __nv_bfloat16* ap = rows[r];
            cp16(&stage_ptr(stage, 0)[r][(i & 3) * 8], ap != nullptr && in_k ? ap + k : a_rows, ap != nullptr && in_k ? 16 : 0);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                bool ok = in_k && n0 + r < F;
                cp16(&stage_ptr(stage, 1 + b)[r][(i & 3) * 8], ok ? wb[b] + (size_t)(n0 + r) * K + k : w, ok ? 16 : 0);
            }
        }
    };
    float acc[NB][32];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[b][i] = 0.f;
    int iters = (K + TILE_K - 1) / TILE_K;
    for (int it = 0; it < PIPE_STAGES - 1; ++it) {
        if (it < iters) issue(it);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    TileBF16 tile;
    for (int it = 0; it < iters; ++it) {
        asm volatile("cp.async.wait_group %0;" ::"n"(PIPE_STAGES - 2) : "memory");
        __syncthreads();
        if (it + PIPE_STAGES - 1 < iters) issue(it + PIPE_STAGES - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        int stage = it % PIPE_STAGES;
        tile.as = stage_ptr(stage, 0);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            tile.bs = stage_ptr(stage, 1 + b);
            tile.mma(acc[b]);
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        int r, c;
        TileBF16::where(i, r, c);
        int pair = pair_of[r];
        if (pair < 0 || n0 + c >= F) continue;
        if constexpr (NB == 2) {
            float g = acc[0][i], u = acc[NB - 1][i];
            if (clamp) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
            y[(size_t)pair * F + n0 + c] = __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + up_offset));
        } else {
            int token = pair / top, choice = pair - token * top;
            out[((size_t)choice * N + token) * F + n0 + c] = weights[pair] * acc[0][i];
        }
    }
}
}  // namespace

IE_API int ie_route_topk(const void* x, int dtype, const float* w, const float* bias, int num_tokens, int width,
                         int experts, int top, int groups, int keep, int sigmoid_scores, const float* correction,
                         int group_top, float weight_scale, int* ids, float* weights, void* stream) {
    if (num_tokens <= 0) return 0;
    if (experts < 1 || groups < 1 || experts % groups || top < 1 || top > experts) return (int)cudaErrorInvalidValue;
    if (group_top < 1 || group_top > 2 || (!sigmoid_scores && (correction != nullptr || group_top != 1)))
        return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)(width + 2 * experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        return ie_launch(route_topk_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(ROUTE_THREADS), smem, s,
                         (const __nv_bfloat16*)x, w, bias, width, experts, top, groups, keep, sigmoid_scores, correction,
                         group_top, weight_scale, ids, weights);
    return ie_launch(route_topk_kernel<float>, dim3(num_tokens), dim3(ROUTE_THREADS), smem, s, (const float*)x, w,
                     bias, width, experts, top, groups, keep, sigmoid_scores, correction, group_top, weight_scale, ids,
                     weights);
}

IE_API int ie_routed_tile_rows() { return TILE_M; }

// The most tiles `pairs` pairs over `experts` experts can need.
IE_API int ie_routed_max_tiles(int pairs, int experts) {
    int used = pairs < experts ? pairs : experts;
    return pairs / TILE_M + used;
}

IE_API int ie_routed_align(const int* ids, int pairs, int experts, int* sorted, int* tile_expert, int* meta,
                           int max_tiles, void* stream) {
    if (pairs <= 0) return 0;
    size_t smem = (size_t)3 * experts * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return ie_launch(routed_align_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, ids, pairs, experts,
                     sorted, tile_expert, meta, max_tiles);
}

IE_API int ie_routed_gate_up(const void* x, const void* w, void* y, int dtype, const int* sorted,
                             const int* tile_expert, const int* meta, int max_tiles, int top, int K, int F,
                             float limit, int clamp, float alpha, float up_offset, void* stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((F + TILE_N - 1) / TILE_N, max_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16 && K % 8 == 0)
        return ie_launch(routed_bf16_kernel<2>, grid, dim3(128), pipe_smem(2), s, (const __nv_bfloat16*)x,
                         (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (float*)nullptr, (const float*)nullptr, sorted,
                         tile_expert, meta, top, 0, K, F, limit, clamp, alpha, up_offset);
    if (dtype == IE_BF16)
        return ie_launch(routed_gate_up_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)x,
                         (const __nv_bfloat16*)w, (__nv_bfloat16*)y, sorted, tile_expert, meta, top, K, F, limit,
                         clamp, alpha, up_offset);
    return ie_launch(routed_gate_up_kernel<float>, grid, dim3(128), 0, s, (const float*)x, (const float*)w,
                     (float*)y, sorted, tile_expert, meta, top, K, F, limit, clamp, alpha, up_offset);
}

IE_API int ie_routed_down(const void* y, const void* w, float* out, const float* weights, int dtype,
                          const int* sorted, const int* tile_expert, const int* meta, int max_tiles, int top,
                          int N, int F, int H, void* stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((H + TILE_N - 1) / TILE_N, max_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16 && F % 8 == 0)
        return ie_launch(routed_bf16_kernel<1>, grid, dim3(128), pipe_smem(1), s, (const __nv_bfloat16*)y,
                         (const __nv_bfloat16*)w, (__nv_bfloat16*)nullptr, out, weights, sorted, tile_expert, meta,
                         top, N, F, H, 0.f, 0, 0.f, 0.f);
    if (dtype == IE_BF16)
        return ie_launch(routed_down_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)y,
                         (const __nv_bfloat16*)w, out, weights, sorted, tile_expert, meta, top, N, F, H);
    return ie_launch(routed_down_kernel<float>, grid, dim3(128), 0, s, (const float*)y, (const float*)w, out,
                     weights, sorted, tile_expert, meta, top, N, F, H);
}
