// Softmax attention with a sink, a sliding window and a gate per head on the tensor cores (bfloat16),
// for prompt portions and single tokens alike.  Built per (key size SK_D, value size SK_DV), both
// multiples of 16.
//
// o_i = gate_i * sum_j p_ij v_j / (sum_j p_ij + exp(sink - m_i)),  p_ij = exp(q_i . k_j * scale - m_i),
// over the keys j with 0 <= i - j < window (window 0: every j <= i).  The sink is one more term of the
// denominator that has no key and no value: a row's running maximum starts at the sink and its running
// sum at 1 (without a sink: -inf and 0).  A block owns 64 consecutive query positions of one request
// and one query head (four warps of 16 rows; warps whose rows do not exist only help to copy); it walks
// the 64-key tiles from the window of its first row to the position of its last row.  Key and value
// tiles come from the request's pages by cp.async into two buffers; S = Q K^T and O += P V by
// mma.sync.m16n8k16 with fragments from ldmatrix (values transposed on the way); scores, maxima, sums
// and the mask are 32-bit, and a weight enters the second product as two bfloat16 terms (its rounded
// value and the remainder), so it keeps 16 bits of mantissa; O stays in registers and is rescaled when
// a row's maximum grows.  A row's result depends on its own request alone (tiles are aligned to
// position 0, keys are added in rising order).
//
// Steps whose requests bring few tokens each (decoding) and whose window is known cut the key tiles
// of a request and head among several blocks (`splits` ranges of `tiles_per_split` tiles, counted from
// the first tile the request's first row sees, so the cut depends on the request's own positions
// alone): each block leaves its unnormalised sums, its running maximum and its running sum in a
// 32-bit scratch row, and a second kernel merges the ranges in rising order, adds the sink's term
// and applies the gate.  Such a block serves all query heads of one key/value head at once: its rows
// are (token, head of the group), so a key tile is brought once for the group.
//
// `softcap` > 0: a score s (after the scale) becomes softcap * tanh(s / softcap) before the softmax.
// `keep_first` > 0 (with a window): the keys at positions below `keep_first` stay visible to every later
// query of the request beside its window, at their own positions.  A block then walks the tiles that
// hold kept keys and lie wholly before its window's first tile, then the window's tiles; with key
// ranges cut among blocks the first `kept_splits` ranges are the kept tiles'.
#include "common.cuh"
#include <math.h>

#ifndef SK_D
#define SK_D 64
#endif
#ifndef SK_DV
#define SK_DV 64
#endif

namespace {
constexpr int D = SK_D, DV = SK_DV;
constexpr int ROWS = 64, KEYS = 64, WARPS = 4, THREADS = WARPS * 32;
static_assert(THREADS == 2 * KEYS, "two threads bring a key's rows");
constexpr int LDK = D + 8, LDV = DV + 8;  // rows 16 bytes longer: ldmatrix rows fall on different banks
static_assert(D % 16 == 0 && DV % 16 == 0 && D <= 256 && DV <= 256, "sizes");
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16z(void* dst, const void* src, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(unsigned* r, const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned* r, const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// tanh from one exponential: 1 - 2 / (e^(2x) + 1), the argument held where tanh is 1 to 32-bit precision
__device__ __forceinline__ float tanh_fast(float x) {
    x = fminf(fmaxf(x, -15.f), 15.f);
    return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);
}
__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

// grid: (query tiles, heads, requests).
__global__ void __launch_bounds__(THREADS)
sink_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                          const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables,
                          int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                          __nv_bfloat16* __restrict__ out, int heads, int kv_heads, int page_size,
                          int total_pages, float scale, int window, const float* __restrict__ sinks,
                          const float* __restrict__ out_gate, int gate_ld, float* __restrict__ partial,
                          int splits, int tiles_per_split, float softcap, int keep_first, int kept_splits,
                          int* err) {
    extern __shared__ __align__(16) unsigned char raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(raw);  // [ROWS][LDK]
    __nv_bfloat16* ks = qs + ROWS * LDK;                        // [2][KEYS][LDK]
    __nv_bfloat16* vs = ks + 2 * KEYS * LDK;                    // [2][KEYS][LDV]
    ie_pdl_trigger();
    ie_pdl_wait();
    // (with `partial` the first grid dimension counts ranges of key tiles and the second key/value heads;
    // row r of the block is then token r / group with query head kvh * group + r % group)
    const bool split_mode = partial != nullptr;
    const int group = heads / kv_heads;
    int seq = blockIdx.z, head = blockIdx.y, tile = split_mode ? 0 : gridDim.x - 1 - blockIdx.x;
    int q0 = cu_q[seq], q_len = cu_q[seq + 1] - q0;
    int row0 = tile * ROWS;
    if (row0 >= q_len) return;
    int tokens_here = min(ROWS, q_len - row0);
    int rows_here = split_mode ? q_len * group : tokens_here;
    int start = ctx_lens[seq] - q_len;  // position of the request's first token of this step
    int first_pos = start + row0, last_pos = first_pos + tokens_here - 1;
    int lo_min = window > 0 ? max(first_pos - window + 1, 0) : 0;
    int kvh = split_mode ? head : head / group;
    // a row's token (counted from the block's first) and query head
    auto row_token = [&](int r) { return split_mode ? r / group : r; };
    auto row_head = [&](int r) { return split_mode ? kvh * group + r % group : head; };
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int* table = block_tables + (size_t)seq * table_width;
    int page_shift = 31 - __clz(page_size);

    // Two threads bring a key's rows (key and value), the 16-byte pieces dealt alternately: one look
    // into the block table per thread and tile, then only copies.
    auto load_tile = [&](int t, int buf) {
        constexpr int KC = D / 8, VC = DV / 8;  // 16-byte pieces of a row
        int key = tid >> 1, pos = t * KEYS + key;
        __nv_bfloat16* kd = ks + ((size_t)buf * KEYS + key) * LDK;
        __nv_bfloat16* vd = vs + ((size_t)buf * KEYS + key) * LDV;
        const __nv_bfloat16* ksrc = k_cache;
        const __nv_bfloat16* vsrc = v_cache;
        int bytes = 0;
        if ((pos >= lo_min || pos < keep_first) && pos <= last_pos) {
            int page = table[pos >> page_shift];
            if (page < 0 || page >= total_pages) {
                if ((tid & 1) == 0) ie_report(err, page < 0 ? IE_ERR_TABLE : IE_ERR_PAGE, page, q0 + row0);
            } else {
                long long row = ((long long)page * kv_heads + kvh) * page_size + (pos & (page_size - 1));
                ksrc = k_cache + row * D;
                vsrc = v_cache + row * DV;
                bytes = 16;
            }
        }
        // (what is outside the range reads as zero: its weight is zero too, and 0 * 0 adds nothing)
#pragma unroll
        for (int c = (tid & 1); c < KC; c += 2) cp_async16z(kd + c * 8, bytes ? ksrc + c * 8 : k_cache, bytes);
#pragma unroll
        for (int c = (tid & 1); c < VC; c += 2) cp_async16z(vd + c * 8, bytes ? vsrc + c * 8 : v_cache, bytes);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // The tiles the block walks, by a running number: first the `kept_tiles` tiles that hold kept keys
    // and lie before the window's first tile (numbers 0 ..), then the window's tiles.
    const int win_begin = lo_min / KEYS, win_end = last_pos / KEYS;  // inclusive
    const int kept_tiles = keep_first > 0 ? min((keep_first - 1) / KEYS + 1, win_begin) : 0;
    auto tile_of = [&](int i) { return i < kept_tiles ? i : win_begin + (i - kept_tiles); };
    int t_begin = 0, t_end = kept_tiles + (win_end - win_begin);  // running numbers, inclusive
    if (split_mode) {
        if ((int)blockIdx.x < kept_splits) {
            t_begin = blockIdx.x * tiles_per_split;
            t_end = min(kept_tiles - 1, t_begin + tiles_per_split - 1);
        } else {
            t_begin = kept_tiles + (blockIdx.x - kept_splits) * tiles_per_split;
            t_end = min(t_end, t_begin + tiles_per_split - 1);
        }
        if (t_begin > t_end) {  // nothing in this range: a maximum of -inf tells the merge to pass over it
            if (tid < rows_here) {
                float* dst = partial + (((size_t)(q0 + row_token(tid)) * heads + row_head(tid)) * splits + blockIdx.x) * (DV + 2);
                dst[DV] = -INFINITY;
                dst[DV + 1] = 0.f;
            }
            return;
        }
    }
    load_tile(tile_of(t_begin), 0);
    // the block's queries (rows beyond the request's tokens read as zero)
    for (int i = tid; i < ROWS * (D / 8); i += THREADS) {
        int r = i / (D / 8), c = i - r * (D / 8);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows_here)
            val = *reinterpret_cast<const uint4*>(q + ((size_t)(q0 + row0 + row_token(r)) * heads + row_head(r)) * D + c * 8);
        *reinterpret_cast<uint4*>(qs + r * LDK + c * 8) = val;
    }
    __syncthreads();
    const bool active = warp * 16 < rows_here;  // (a warp without rows copies tiles and waits at the barriers)
    unsigned qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldsm_x4(qf[kk], qs + (warp * 16 + (lane & 15)) * LDK + kk * 16 + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // the two rows of this thread: positions and the first position each may see
    int r_a = warp * 16 + g, r_b = r_a + 8;
    int pos_a = r_a < rows_here ? first_pos + row_token(r_a) : -1, pos_b = r_b < rows_here ? first_pos + row_token(r_b) : -1;
    int lo_a = window > 0 ? max(pos_a - window + 1, 0) : 0;
    int lo_b = window > 0 ? max(pos_b - window + 1, 0) : 0;
    // running maximum (of score * scale * log2 e) and this thread's share of the running sum; the
    // sink's term of the sum is counted by the first thread of the four that share a row
    const float sl2 = scale * LOG2E;
    const float cap_in = softcap > 0.f ? scale / softcap : 0.f, cap_out = softcap * LOG2E;
    const bool with_sink = sinks != nullptr && !split_mode;  // (split: the merge adds the sink's term)
    float sink2 = with_sink ? sinks[head] * LOG2E : -INFINITY;
    float m_a = sink2, m_b = sink2;
    float l_a = (with_sink && t4 == 0) ? 1.f : 0.f, l_b = l_a;

    int buf = 0;
    for (int ti = t_begin; ti <= t_end; ++ti, buf ^= 1) {
        const int t = tile_of(ti);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // the tile has landed for everyone, and everyone is done with the other buffer
        if (ti < t_end) load_tile(tile_of(ti + 1), buf ^ 1);
        if (!active) continue;
        const __nv_bfloat16* kt = ks + (size_t)buf * KEYS * LDK;
        const __nv_bfloat16* vt = vs + (size_t)buf * KEYS * LDV;
        float s[KEYS / 8][4];
#pragma unroll
        for (int i = 0; i < KEYS / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int nt = 0; nt < KEYS / 8; nt += 2) {
                unsigned b[4];  // keys nt * 8 .. + 15: (entries kk * 16 .. + 7, .. + 15) of each eight
                ldsm_x4(b, kt + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[nt], qf[kk], b[0], b[1]);
                mma_bf16(s[nt + 1], qf[kk], b[2], b[3]);
            }
        }
        // scores in units of log2 e, -inf where the key is not visible; the rows' new maxima
        float mx_a = m_a, mx_b = m_b;
#pragma unroll
        for (int nt = 0; nt < KEYS / 8; ++nt) {
            int kp = t * KEYS + nt * 8 + t4 * 2;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int key_pos = kp + (e & 1);
                int pos = e < 2 ? pos_a : pos_b, lo = e < 2 ? lo_a : lo_b;
                bool visible = key_pos <= pos && (key_pos >= lo || key_pos < keep_first);
                float sc = softcap > 0.f ? cap_out * tanh_fast(s[nt][e] * cap_in) : s[nt][e] * sl2;
                s[nt][e] = visible ? sc : -INFINITY;
            }
            mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
        }
        mx_a = quad_max(mx_a);
        mx_b = quad_max(mx_b);
        // (a row that has seen nothing yet keeps -inf: its factor and its weights are zero)
        float al_a = m_a == -INFINITY ? 0.f : exp2f(m_a - mx_a), al_b = m_b == -INFINITY ? 0.f : exp2f(m_b - mx_b);
        float sub_a = mx_a == -INFINITY ? 0.f : mx_a, sub_b = mx_b == -INFINITY ? 0.f : mx_b;
        m_a = mx_a;
        m_b = mx_b;
        if (al_a != 1.f || al_b != 1.f) {
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
            }
        }
        float sum_a = 0.f, sum_b = 0.f;
        unsigned pf[KEYS / 16][4], pl[KEYS / 16][4];
#pragma unroll
        for (int nt = 0; nt < KEYS / 8; ++nt) {
            float w[4];
            w[0] = exp2f(s[nt][0] - sub_a);  // (exp2 of -inf is 0)
            w[1] = exp2f(s[nt][1] - sub_a);
            w[2] = exp2f(s[nt][2] - sub_b);
            w[3] = exp2f(s[nt][3] - sub_b);
            sum_a += w[0] + w[1];
            sum_b += w[2] + w[3];
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16(w[0], w[1]);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(w[2], w[3]);
            pl[nt >> 1][(nt & 1) * 2] = pack_bf16(w[0] - bf16_round(w[0]), w[1] - bf16_round(w[1]));
            pl[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(w[2] - bf16_round(w[2]), w[3] - bf16_round(w[3]));
        }
        l_a = l_a * al_a + sum_a;
        l_b = l_b * al_b + sum_b;
#pragma unroll
        for (int kk = 0; kk < KEYS / 16; ++kk) {
#pragma unroll
            for (int nt = 0; nt < DV / 8; nt += 2) {
                unsigned b[4];  // keys kk * 16 .. + 15 of value columns nt * 8 .. + 15, transposed
                ldsm_x4_trans(b, vt + (kk * 16 + (lane & 15)) * LDV + nt * 8 + (lane >> 4) * 8);
                mma_bf16(o[nt], pf[kk], b[0], b[1]);
                mma_bf16(o[nt + 1], pf[kk], b[2], b[3]);
                mma_bf16(o[nt], pl[kk], b[0], b[1]);
                mma_bf16(o[nt + 1], pl[kk], b[2], b[3]);
            }
        }
    }
    if (!active) return;
    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    if (split_mode) {
        float* dst_a = partial + (((size_t)(q0 + row_token(r_a)) * heads + row_head(r_a)) * splits + blockIdx.x) * (DV + 2);
        float* dst_b = partial + (((size_t)(q0 + row_token(r_b)) * heads + row_head(r_b)) * splits + blockIdx.x) * (DV + 2);
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            int c = nt * 8 + t4 * 2;
            if (pos_a >= 0) *reinterpret_cast<float2*>(dst_a + c) = make_float2(o[nt][0], o[nt][1]);
            if (pos_b >= 0) *reinterpret_cast<float2*>(dst_b + c) = make_float2(o[nt][2], o[nt][3]);
        }
        if (t4 == 0) {
            if (pos_a >= 0) { dst_a[DV] = m_a; dst_a[DV + 1] = l_a; }
            if (pos_b >= 0) { dst_b[DV] = m_b; dst_b[DV + 1] = l_b; }
        }
        return;
    }
    float f_a = l_a > 0.f ? 1.0f / l_a : 0.f, f_b = l_b > 0.f ? 1.0f / l_b : 0.f;
    if (out_gate != nullptr) {
        if (pos_a >= 0) f_a *= 1.0f / (1.0f + expf(-out_gate[(size_t)(q0 + row0 + r_a) * gate_ld + head]));
        if (pos_b >= 0) f_b *= 1.0f / (1.0f + expf(-out_gate[(size_t)(q0 + row0 + r_b) * gate_ld + head]));
    }
    __nv_bfloat16* out_a = out + ((size_t)(q0 + row0 + r_a) * heads + head) * DV;
    __nv_bfloat16* out_b = out + ((size_t)(q0 + row0 + r_b) * heads + head) * DV;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
        int c = nt * 8 + t4 * 2;
        if (pos_a >= 0) *reinterpret_cast<unsigned*>(out_a + c) = pack_bf16(o[nt][0] * f_a, o[nt][1] * f_a);
        if (pos_b >= 0) *reinterpret_cast<unsigned*>(out_b + c) = pack_bf16(o[nt][2] * f_b, o[nt][3] * f_b);
    }
}

constexpr int MERGE_MAX_SPLITS = 1024;
// grid: tokens * heads.  Merges a token and head's ranges in rising order: maxima and sums are in units
// of log2 e; the sink (if any) is one more term of the sum; the gate multiplies the result.
__global__ void __launch_bounds__(128)
sink_attention_merge_kernel(const float* __restrict__ partial, const int* __restrict__ cu_q, int num_seqs,
                            __nv_bfloat16* __restrict__ out, int heads, int splits,
                            const float* __restrict__ sinks, const float* __restrict__ out_gate, int gate_ld) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int token = blockIdx.x / heads, head = blockIdx.x - token * heads;
    if (token >= cu_q[num_seqs]) return;  // (a captured step's padding belongs to no request)
    const float* src = partial + ((size_t)token * heads + head) * splits * (DV + 2);
    // the ranges' maxima and sums first, all at once (a range per thread), then the rows
    __shared__ float s_m[MERGE_MAX_SPLITS], s_l[MERGE_MAX_SPLITS];
    for (int s = threadIdx.x; s < splits; s += 128) {
        s_m[s] = src[(size_t)s * (DV + 2) + DV];
        s_l[s] = src[(size_t)s * (DV + 2) + DV + 1];
    }
    __syncthreads();
    float m = sinks != nullptr ? sinks[head] * LOG2E : -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, s_m[s]);
    float l = sinks != nullptr ? exp2f(sinks[head] * LOG2E - m) : 0.f;
    if (m == -INFINITY) m = 0.f;
    float acc[(DV + 127) / 128];
#pragma unroll
    for (int i = 0; i < (DV + 127) / 128; ++i) acc[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
        const float* row = src + (size_t)s * (DV + 2);
        float ms = s_m[s];
        bool empty = ms == -INFINITY;  // (an empty range: its sums were never written)
        float w = empty ? 0.f : exp2f(ms - m);
        l = fmaf(s_l[s], w, l);
#pragma unroll
        for (int i = 0; i < (DV + 127) / 128; ++i) {
            int c = i * 128 + threadIdx.x;
            float v = (c < DV && !empty) ? row[c] : 0.f;
            acc[i] = fmaf(v, w, acc[i]);
        }
    }
    float f = l > 0.f ? 1.0f / l : 0.f;
    if (out_gate != nullptr) f *= 1.0f / (1.0f + expf(-out_gate[(size_t)token * gate_ld + head]));
#pragma unroll
    for (int i = 0; i < (DV + 127) / 128; ++i) {
        int c = i * 128 + threadIdx.x;
        if (c < DV) out[((size_t)token * heads + head) * DV + c] = __float2bfloat16_rn(acc[i] * f);
    }
}
}  // namespace

IE_API int ie_sink_attention_dims(int* d, int* dv) {
    *d = D;
    *dv = DV;
    return 0;
}

IE_API int ie_sink_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                 int table_width, const int* cu_q, const int* ctx_lens, void* out, int num_seqs,
                                 int max_q_len, int heads, int kv_heads, int page_size, int total_pages,
                                 float scale, int window, const float* sinks, const float* out_gate, int gate_ld,
                                 float* partial, int splits, int tiles_per_split, int num_tokens, float softcap,
                                 int keep_first, int kept_splits, int* err, void* stream) {
    if (num_seqs <= 0 || max_q_len <= 0) return 0;
    if (kv_heads <= 0 || heads % kv_heads != 0 || page_size < 1 || (page_size & (page_size - 1)) || window < 0)
        return (int)cudaErrorInvalidValue;
    if (softcap < 0.f || keep_first < 0 || kept_splits < 0 || (window == 0 && keep_first > 0))
        return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)(ROWS * LDK + 2 * KEYS * LDK + 2 * KEYS * LDV) * sizeof(__nv_bfloat16);
    static IePerDevice allowed;
    cudaError_t e = ie_allow_smem(allowed, sink_attention_mma_kernel, smem);
    if (e != cudaSuccess) return (int)e;
    if (partial != nullptr) {
        // ranges of key tiles: a request's tokens times the heads of a group are one tile of rows, and
        // the scratch holds [num_tokens, heads, splits, DV + 2] floats
        if (max_q_len * (heads / kv_heads) > ROWS || splits < 1 || splits > MERGE_MAX_SPLITS || tiles_per_split < 1 ||
            num_tokens < 1 || kept_splits >= splits)
            return (int)cudaErrorInvalidValue;
        int rc = ie_launch(sink_attention_mma_kernel, dim3(splits, kv_heads, num_seqs), dim3(THREADS), smem,
                           (cudaStream_t)stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                           (const __nv_bfloat16*)v_cache, block_tables, table_width, cu_q, ctx_lens, (__nv_bfloat16*)out,
                           heads, kv_heads, page_size, total_pages, scale, window, sinks, out_gate, gate_ld, partial,
                           splits, tiles_per_split, softcap, keep_first, kept_splits, err);
        if (rc != 0) return rc;
        return ie_launch(sink_attention_merge_kernel, dim3(num_tokens * heads), dim3(128), 0, (cudaStream_t)stream,
                         (const float*)partial, cu_q, num_seqs, (__nv_bfloat16*)out, heads, splits, sinks, out_gate,
                         gate_ld);
    }
    dim3 grid((max_q_len + ROWS - 1) / ROWS, heads, num_seqs);
    return ie_launch(sink_attention_mma_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream,
                     (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables,
                     table_width, cu_q, ctx_lens, (__nv_bfloat16*)out, heads, kv_heads, page_size, total_pages, scale,
                     window, sinks, out_gate, gate_ld, (float*)nullptr, 1, 0, softcap, keep_first, 0, err);
}
