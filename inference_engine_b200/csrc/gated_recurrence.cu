// Kernels of recurrent mixers whose state is a matrix per head that decays and takes an outer
// product per token:   S_t = diag(a_t) S_(t-1) + w_t u_t^T,   o_t = S_t^T q_t,
// with S of dim x cols (32-bit, kept column by column in the request's state slot).
//
//  * gated-write linear attention (HGRN2): a_t = f_t and w_t = 1 - f_t per head and channel,
//    u_t = v_t, f_t = lower + (1 - lower) * sigmoid(. + bias); q_t = silu(.).
//  * matrix memory with exponential gates (mLSTM): a_t and a write gate b_t are one number per
//    head, w_t = k_t, u_t = b_t v_t, and one more column whose value is 1 carries the
//    normaliser n_t = a_t n_(t-1) + b_t k_t.  The gates come from a running maximum m_t that
//    starts at 0:  m_t = max(logf_t + m_(t-1), logi_t),  a_t = exp(logf_t + m_(t-1) - m_t),
//    b_t = exp(logi_t - m_t);  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).
//
//  * gated linear attention: a_t per head and channel from a low-rank map of the input,
//    a_t = sigmoid(z_t)^(1 / tau) with z_t = W2 y_t + b (y_t the input's projection to a few
//    numbers), taken as exp(logsigmoid(z_t) / tau); w_t = k_t, u_t = v_t; the read-out's gate is
//    silu(.) instead of sigmoid(.).
//
// Kernels: lowrank_decay (a block takes sixteen tokens and 128 channels, so that a row of W2 is read
// once per sixteen tokens); short_conv_residual (+ tail update): out = x + causal convolution of x over time per
// channel, the last taps - 1 inputs kept per request; hgrn2_gates; mlstm_gates (a warp per request
// and head walks the step's tokens in order); gated_recurrence (columns of S do not interact: a
// block owns some columns of one head of one request, TPC lanes a column, tokens in order, eight at
// a time through a ring of four shared-memory buffers, three chunks on their way); recurrence_readout (normaliser,
// unit root mean square per head, weight, output gate).  Every sum is taken in an order that
// depends on the sizes alone, never on how a request's tokens were cut into steps or batched.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ float silu_f(float y) { return y / (1.0f + expf(-y)); }
__device__ __forceinline__ float sigmoid_f(float y) { return 1.0f / (1.0f + expf(-y)); }
__device__ __forceinline__ float logsigmoid_f(float y) { return fminf(y, 0.f) - log1pf(expf(-fabsf(y))); }

// grid: (tokens, blocks of channels).  x and out: [N, channels] in the compute dtype; w: [channels, taps], the last tap
// weighs the token itself; tail: the slot's kept inputs [taps - 1][channels], oldest first.
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_residual_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ state,
                           long long state_stride, const int* __restrict__ slots,
                           const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                           T* __restrict__ out, int channels, int taps, int num_slots, int* err) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x;
    int seq = seq_of_token[n];
    int t = n - cu_q[seq];
    int slot = slots[seq];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) ie_report(err, IE_ERR_PAGE, slot, n);
        return;
    }
    const float* tail = state + (size_t)slot * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            int back = taps - 1 - j;
            float xv = (t - back >= 0) ? ie_load(x + (size_t)(n - back) * channels + c)
                                       : tail[(size_t)(taps - 1 + t - back) * channels + c];
            acc = fmaf(w[(size_t)c * taps + j], xv, acc);
        }
        ie_store(out + (size_t)n * channels + c, ie_load(x + (size_t)n * channels + c) + acc);
    }
}

// grid: (requests of the step, blocks of channels): the kept inputs become the last taps - 1 of (kept, new).
template <typename T>
__global__ void short_conv_tail_kernel(const T* __restrict__ x, float* __restrict__ state, long long state_stride,
                                       const int* __restrict__ slots, const int* __restrict__ cu_q, int channels,
                                       int taps, int num_slots) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int seq = blockIdx.x;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    float* tail = state + (size_t)slot * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        // a thread owns a channel and goes through the rows in rising order, so a kept row is
        // read before it is overwritten
        for (int j = 0; j < taps - 1; ++j) {
            int tt = len - (taps - 1) + j;
            float xv = tt >= 0 ? ie_load(x + (size_t)(start + tt) * channels + c)
                               : tail[(size_t)(taps - 1 + tt) * channels + c];
            tail[(size_t)j * channels + c] = xv;
        }
    }
}

// proj: [N, ld] 32-bit, columns q (size), forget pre-activations (size), then whatever follows.
// In place: q <- silu(q), f <- lower + (1 - lower) * sigmoid(f + bias); write[n, c] = 1 - f.
__global__ void hgrn2_gates_kernel(float* __restrict__ proj, int ld, const float* __restrict__ bias,
                                   const float* __restrict__ lower, float* __restrict__ write, int size,
                                   size_t total) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        size_t n = idx / size;
        int c = (int)(idx - n * size);
        float* row = proj + n * ld;
        row[c] = silu_f(row[c]);
        float l = lower[c];
        float f = l + (1.0f - l) * sigmoid_f(row[size + c] + bias[c]);
        row[size + c] = f;
        write[idx] = 1.0f - f;
    }
}

// grid: (heads, requests), one warp each.  gi, gf: the gates' pre-activations, element (n, head) at
// [n * ld + head].  gates: [N, heads, 3] = (a, b, exp(-m)).  m: the running maximum of a head,
// in the slot at `m_offset + head`.
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const float* __restrict__ gi, const float* __restrict__ gf, int ld,
                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                   float* __restrict__ state, long long state_stride, long long m_offset,
                   const int* __restrict__ slots, const int* __restrict__ cu_q, float* __restrict__ gates,
                   int heads, int num_slots) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int head = blockIdx.x, seq = blockIdx.y, lane = threadIdx.x;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    float* m_ptr = state + (size_t)slot * state_stride + m_offset + head;
    float m = *m_ptr;
    float bi = bias_i[head], bf = bias_f[head];
    for (int t0 = 0; t0 < len; t0 += 32) {
        int cnt = min(32, len - t0);
        float li = 0.f, lf = 0.f;
        if (lane < cnt) {
            size_t n = (size_t)(start + t0 + lane);
            li = cap * tanhf((gi[n * ld + head] + bi) / cap);
            lf = logsigmoid_f(cap * tanhf((gf[n * ld + head] + bf) / cap));
        }
        float m_before = 0.f, m_mine = 0.f;
        for (int j = 0; j < cnt; ++j) {  // the chain, the same in every lane
            float fj = __shfl_sync(0xffffffffu, lf, j), ij = __shfl_sync(0xffffffffu, li, j);
            float m_new = fmaxf(fj + m, ij);
            if (lane == j) { m_before = m; m_mine = m_new; }
            m = m_new;
        }
        if (lane < cnt) {
            float* g = gates + ((size_t)(start + t0 + lane) * heads + head) * 3;
            g[0] = expf(lf + m_before - m_mine);
            g[1] = expf(li - m_mine);
            g[2] = expf(-m_mine);
        }
    }
    if (lane == 0) *m_ptr = m;
}

// grid: (blocks of LD_TOKENS tokens, blocks of 128 channels).  y: element (n, r) at [n * y_ld + r]; w2: [channels, rank];
// decay: [N, channels] = exp(logsigmoid(w2 y + bias) * inv_tau).  A channel's sum runs over r in rising order.
// The block's 128 rows of w2 and its tokens' inputs pass through shared memory 32 ranks at a time: a warp
// reads 32 consecutive numbers of a row at once, and rows sit 33 words apart so that the threads of a
// warp, one channel each, read different banks.
constexpr int LD_TOKENS = 16, LD_RANKS = 32;
__global__ void __launch_bounds__(128)
lowrank_decay_kernel(const float* __restrict__ y, int y_ld, const float* __restrict__ w2,
                     const float* __restrict__ bias, float inv_tau, float* __restrict__ decay, int num_tokens,
                     int channels, int rank) {
    __shared__ float ws[128 * (LD_RANKS + 1)];
    __shared__ float ys[LD_TOKENS * LD_RANKS];
    ie_pdl_trigger();
    ie_pdl_wait();
    int n0 = blockIdx.x * LD_TOKENS, c0 = blockIdx.y * 128;
    int cnt = min(LD_TOKENS, num_tokens - n0);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc[LD_TOKENS];
#pragma unroll
    for (int t = 0; t < LD_TOKENS; ++t) acc[t] = 0.f;
    for (int r0 = 0; r0 < rank; r0 += LD_RANKS) {
        int width = min(LD_RANKS, rank - r0);
        if (r0 > 0) __syncthreads();  // everyone is done with the last piece
        for (int row = warp; row < 128; row += 4) {
            int c = c0 + row;
            ws[row * (LD_RANKS + 1) + lane] = (c < channels && lane < width) ? w2[(size_t)c * rank + r0 + lane] : 0.f;
        }
        for (int t = warp; t < LD_TOKENS; t += 4)
            ys[t * LD_RANKS + lane] = (t < cnt && lane < width) ? y[(size_t)(n0 + t) * y_ld + r0 + lane] : 0.f;
        __syncthreads();
        const float* wrow = ws + threadIdx.x * (LD_RANKS + 1);
        for (int r = 0; r < width; ++r) {
            float wv = wrow[r];
#pragma unroll
            for (int t = 0; t < LD_TOKENS; ++t) acc[t] = fmaf(wv, ys[t * LD_RANKS + r], acc[t]);
        }
    }
    int c = c0 + threadIdx.x;
    if (c >= channels) return;
    float b = bias != nullptr ? bias[c] : 0.f;
#pragma unroll
    for (int t = 0; t < LD_TOKENS; ++t)
        if (t < cnt) decay[(size_t)(n0 + t) * channels + c] = expf(logsigmoid_f(acc[t] + b) * inv_tau);
}

constexpr int GR_THREADS = 128;
constexpr int GR_CHUNK = 8;  // tokens staged in shared memory at a time
constexpr int GR_STAGES = 4;  // ... in a ring of so many buffers: three chunks are on their way while one is worked on

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// grid: (column blocks, heads, requests).  Lane `sub` of a column's TPC lanes holds rows sub, sub + TPC,
// ..., R of them.  q, a, w: element (n, head, d) at [n * ld + head * dim + d]; SCALAR: a and the write
// gate b come from gates[(n * heads + head) * 3 + {0, 1}] and column `vdim` (if cols > vdim) has the
// value 1.  v: (n, head, c) at [n * v_ld + head * vdim + c].  out: [N, heads, cols], times q_scale.
template <int R, int TPC, bool SCALAR>
__global__ void __launch_bounds__(GR_THREADS)
gated_recurrence_kernel(const float* __restrict__ q, int q_ld, const float* __restrict__ a, int a_ld,
                        const float* __restrict__ w, int w_ld, const float* __restrict__ gates,
                        const float* __restrict__ v, int v_ld, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ slots, const int* __restrict__ cu_q, float* __restrict__ out,
                        int heads, int dim, int vdim, int cols, float q_scale, int num_slots) {
    extern __shared__ __align__(16) float sm[];
    constexpr int COLS = GR_THREADS / TPC, DP = R * TPC;
    constexpr int ROWS = SCALAR ? 2 : 3;  // arrays of DP floats per token: q, w (, a)
    constexpr int BUF = GR_CHUNK * (ROWS * DP + COLS + 4);
    ie_pdl_trigger();
    ie_pdl_wait();
    int seq = blockIdx.z, head = blockIdx.y;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    int tid = threadIdx.x;
    int sub = tid % TPC, my_col = tid / TPC, col = blockIdx.x * COLS + my_col;
    bool live = col < cols;
    float* S = state + (size_t)slot * state_stride + ((size_t)head * cols + (live ? col : 0)) * dim;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        int r = sub + TPC * i;
        s[i] = (live && r < dim) ? S[r] : 0.f;
    }
    // entries beyond dim (the copies never touch them) read as zero
    if (DP > dim) {
        int pad = DP - dim;
        for (int i = tid; i < GR_STAGES * GR_CHUNK * ROWS * pad; i += GR_THREADS) {
            int row = i / pad, c = dim + (i - row * pad);
            sm[(row / (GR_CHUNK * ROWS)) * BUF + (row % (GR_CHUNK * ROWS)) * DP + c] = 0.f;
        }
    }
    __syncthreads();
    int c0 = blockIdx.x * COLS;
    bool vec = (dim % 4 == 0) && (q_ld % 4 == 0) && (w_ld % 4 == 0) && (SCALAR || a_ld % 4 == 0) &&
               ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(w) |
                 (SCALAR ? 0 : reinterpret_cast<uintptr_t>(a))) % 16 == 0);
    auto stage = [&](int t0, int b) {
        int cnt = min(GR_CHUNK, len - t0);
        float* qs = sm + b * BUF;
        float* ws = qs + GR_CHUNK * DP;
        float* as = ws + GR_CHUNK * DP;  // (SCALAR: not there; vs starts here)
        float* vs = sm + b * BUF + ROWS * GR_CHUNK * DP;
        float* gs = vs + GR_CHUNK * COLS;  // a and b of the tokens (SCALAR)
        if (vec) {
            int dq = dim >> 2;
            for (int i = tid; i < cnt * dq; i += GR_THREADS) {
                int tt = i / dq, d = (i - tt * dq) * 4;
                size_t n = (size_t)(start + t0 + tt);
                cp_async16(qs + tt * DP + d, q + n * q_ld + head * dim + d);
                cp_async16(ws + tt * DP + d, w + n * w_ld + head * dim + d);
                if (!SCALAR) cp_async16(as + tt * DP + d, a + n * a_ld + head * dim + d);
            }
        } else {
            for (int i = tid; i < cnt * dim; i += GR_THREADS) {
                int tt = i / dim, d = i - tt * dim;
                size_t n = (size_t)(start + t0 + tt);
                cp_async4(qs + tt * DP + d, q + n * q_ld + head * dim + d);
                cp_async4(ws + tt * DP + d, w + n * w_ld + head * dim + d);
                if (!SCALAR) cp_async4(as + tt * DP + d, a + n * a_ld + head * dim + d);
            }
        }
        for (int i = tid; i < cnt * COLS; i += GR_THREADS) {
            int tt = i / COLS, c = i - tt * COLS;
            if (c0 + c < vdim) cp_async4(vs + tt * COLS + c, v + (size_t)(start + t0 + tt) * v_ld + head * vdim + c0 + c);
        }
        if (SCALAR && tid < 2 * cnt)
            cp_async4(gs + tid, gates + ((size_t)(start + t0 + (tid >> 1)) * heads + head) * 3 + (tid & 1));
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // (a step of one chunk waits for its memory once; a prompt's chunks find theirs landed: with one
    // chunk ahead every eight tokens cost a trip to memory, 0.25 us a token whatever the sizes)
    int n_chunks = (len + GR_CHUNK - 1) / GR_CHUNK;
    for (int c = 0; c < GR_STAGES - 1; ++c) {
        if (c < n_chunks) stage(c * GR_CHUNK, c);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    bool ones = SCALAR && live && col >= vdim;  // the normaliser's column
    for (int c = 0; c < n_chunks; ++c) {
        int t0 = c * GR_CHUNK, b = c % GR_STAGES;
        int cnt = min(GR_CHUNK, len - t0);
        asm volatile("cp.async.wait_group %0;" ::"n"(GR_STAGES - 2) : "memory");
        __syncthreads();  // this chunk has landed for everyone, and everyone is done with the buffer filled next
        if (c + GR_STAGES - 1 < n_chunks) stage((c + GR_STAGES - 1) * GR_CHUNK, (c + GR_STAGES - 1) % GR_STAGES);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const float* qs = sm + b * BUF + sub;
        const float* ws = qs + GR_CHUNK * DP;
        const float* as = ws + GR_CHUNK * DP;
        const float* vs = sm + b * BUF + ROWS * GR_CHUNK * DP + my_col;
        const float* gs = sm + b * BUF + ROWS * GR_CHUNK * DP + GR_CHUNK * COLS;
        // The chunk's tokens in order; their read-outs are summed over a column's lanes together at the
        // end, so that the exchanges of eight tokens overlap instead of each stalling the next token.
        float rds[GR_CHUNK];
#pragma unroll
        for (int tt = 0; tt < GR_CHUNK; ++tt) {
            rds[tt] = 0.f;
            if (tt < cnt) {
                float u = ones ? 1.0f : (live ? vs[tt * COLS] : 0.f);
                float a_s = 1.0f;
                if (SCALAR) { a_s = gs[2 * tt]; u *= gs[2 * tt + 1]; }
                float r4[4] = {0.f, 0.f, 0.f, 0.f};  // four partial sums: shorter chains, a fixed order
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    int at = tt * DP + TPC * i;
                    float av = SCALAR ? a_s : as[at];
                    s[i] = fmaf(ws[at], u, s[i] * av);
                    r4[i & 3] = fmaf(s[i], qs[at], r4[i & 3]);
                }
                rds[tt] = (r4[0] + r4[1]) + (r4[2] + r4[3]);
            }
        }
#pragma unroll
        for (int o = TPC >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int tt = 0; tt < GR_CHUNK; ++tt) rds[tt] += __shfl_xor_sync(0xffffffffu, rds[tt], o);
        }
        if (live && sub == 0) {
#pragma unroll
            for (int tt = 0; tt < GR_CHUNK; ++tt)
                if (tt < cnt) out[((size_t)(start + t0 + tt) * heads + head) * cols + col] = rds[tt] * q_scale;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            int r = sub + TPC * i;
            if (r < dim) S[r] = s[i];
        }
    }
}

// One warp per (token, head).  o: [rows, cols]; with `gates` the column `vdim` is n . q and the
// row is first divided by max(|n . q|, exp(-m)) + 1e-6.  weight: [vdim] shared by the heads, or
// [heads * vdim].  gate_pre (optional): element (n, head, d) at [n * gate_ld + head * vdim + d]; the
// row is multiplied by sigmoid(gate_pre), or by silu(gate_pre) with gate_silu.
template <typename T>
__global__ void __launch_bounds__(128)
recurrence_readout_kernel(const float* __restrict__ o, int cols, const float* __restrict__ gates,
                          const float* __restrict__ weight, int weight_per_head, float eps,
                          const float* __restrict__ gate_pre, int gate_ld, int gate_silu, T* __restrict__ out,
                          long long rows, int heads, int vdim) {
    ie_pdl_trigger();
    ie_pdl_wait();
    long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    long long n = row / heads;
    int head = (int)(row - n * heads);
    const float* src = o + row * cols;
    float den = 1.0f;
    if (gates != nullptr) den = fmaxf(fabsf(src[vdim]), gates[row * 3 + 2]) + 1e-6f;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) {
        float x = src[d] / den;
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const float* wrow = weight + (weight_per_head ? (size_t)head * vdim : 0);
    for (int d = lane; d < vdim; d += 32) {
        float y = (src[d] / den) * inv * wrow[d];
        if (gate_pre != nullptr) {
            float gp = gate_pre[n * gate_ld + (size_t)head * vdim + d];
            y *= gate_silu ? silu_f(gp) : sigmoid_f(gp);
        }
        ie_store(out + row * vdim + d, y);
    }
}

inline int grid_for(size_t total, int threads) {
    size_t want = (total + threads - 1) / threads;
    return (int)(want < 148 * 16 ? want : 148 * 16);
}

template <int R, int TPC, bool SCALAR>
int launch_recurrence(const float* q, int q_ld, const float* a, int a_ld, const float* w, int w_ld,
                      const float* gates, const float* v, int v_ld, float* state, long long state_stride,
                      const int* slots, const int* cu_q, float* out, int num_seqs, int heads, int dim, int vdim,
                      int cols, float q_scale, int num_slots, cudaStream_t s) {
    constexpr int COLS = GR_THREADS / TPC;
    size_t smem = (size_t)GR_STAGES * GR_CHUNK * ((SCALAR ? 2 : 3) * R * TPC + COLS + 4) * sizeof(float);
    static IePerDevice allowed;
    cudaError_t e = ie_allow_smem(allowed, gated_recurrence_kernel<R, TPC, SCALAR>, 200 * 1024);  // (dim 512: 198 KB)
    if (e != cudaSuccess) return (int)e;
    dim3 grid((cols + COLS - 1) / COLS, heads, num_seqs);
    return ie_launch(gated_recurrence_kernel<R, TPC, SCALAR>, grid, dim3(GR_THREADS), smem, s, q, q_ld, a, a_ld, w,
                     w_ld, gates, v, v_ld, state, state_stride, slots, cu_q, out, heads, dim, vdim, cols, q_scale,
                     num_slots);
}
}  // namespace

IE_API int ie_short_conv_residual(const void* x, int dtype, const float* w, float* state, long long state_stride,
                                  const int* slots, const int* seq_of_token, const int* cu_q, void* out,
                                  int num_tokens, int num_seqs, int channels, int taps, int num_slots, int* err,
                                  void* stream) {
    if (num_tokens <= 0) return 0;
    if (taps < 1) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    int e;
    // few tokens: a thread per channel; many: a few channels per thread
    int per_row = (channels + 255) / 256;
    int cb = num_tokens >= 512 ? (per_row < 2 ? per_row : 2) : per_row;
    dim3 grid(num_tokens, cb), tail_grid(num_seqs, per_row);
    if (dtype == IE_BF16)
        e = ie_launch(short_conv_residual_kernel<__nv_bfloat16>, grid, dim3(256), 0, s,
                      (const __nv_bfloat16*)x, w, (const float*)state, state_stride, slots, seq_of_token, cu_q,
                      (__nv_bfloat16*)out, channels, taps, num_slots, err);
    else
        e = ie_launch(short_conv_residual_kernel<float>, grid, dim3(256), 0, s, (const float*)x, w,
                      (const float*)state, state_stride, slots, seq_of_token, cu_q, (float*)out, channels, taps,
                      num_slots, err);
    if (e != 0 || taps < 2) return e;
    if (dtype == IE_BF16)
        return ie_launch(short_conv_tail_kernel<__nv_bfloat16>, tail_grid, dim3(256), 0, s,
                         (const __nv_bfloat16*)x, state, state_stride, slots, cu_q, channels, taps, num_slots);
    return ie_launch(short_conv_tail_kernel<float>, tail_grid, dim3(256), 0, s, (const float*)x, state,
                     state_stride, slots, cu_q, channels, taps, num_slots);
}

IE_API int ie_lowrank_decay(const float* y, int y_ld, const float* w2, const float* bias, float inv_tau,
                            float* decay, int num_tokens, int channels, int rank, void* stream) {
    if (num_tokens <= 0 || channels <= 0) return 0;
    if (rank < 1) return (int)cudaErrorInvalidValue;
    dim3 grid((num_tokens + LD_TOKENS - 1) / LD_TOKENS, (channels + 127) / 128);
    return ie_launch(lowrank_decay_kernel, grid, dim3(128), 0, (cudaStream_t)stream, y, y_ld, w2, bias, inv_tau,
                     decay, num_tokens, channels, rank);
}

IE_API int ie_hgrn2_gates(float* proj, int ld, const float* bias, const float* lower, float* write,
                          int num_tokens, int size, void* stream) {
    size_t total = (size_t)num_tokens * size;
    if (total == 0) return 0;
    return ie_launch(hgrn2_gates_kernel, dim3(grid_for(total, 256)), dim3(256), 0, (cudaStream_t)stream, proj, ld,
                     bias, lower, write, size, total);
}

IE_API int ie_mlstm_gates(const float* gi, const float* gf, int ld, const float* bias_i, const float* bias_f,
                          float cap, float* state, long long state_stride, long long m_offset, const int* slots,
                          const int* cu_q, float* gates, int num_seqs, int heads, int num_slots, void* stream) {
    if (num_seqs <= 0 || heads <= 0) return 0;
    return ie_launch(mlstm_gates_kernel, dim3(heads, num_seqs), dim3(32), 0, (cudaStream_t)stream, gi, gf, ld,
                     bias_i, bias_f, cap, state, state_stride, m_offset, slots, cu_q, gates, heads, num_slots);
}

// gates == nullptr: a and w per head and channel (a, a_ld given); else the gates' scalars.
IE_API int ie_gated_recurrence(const float* q, int q_ld, const float* a, int a_ld, const float* w, int w_ld,
                               const float* gates, const float* v, int v_ld, float* state, long long state_stride,
                               const int* slots, const int* cu_q, float* out, int num_seqs, int heads, int dim,
                               int vdim, int cols, float q_scale, int num_slots, void* stream) {
    if (num_seqs <= 0) return 0;
    if (cols < vdim || cols > vdim + 1 || (gates == nullptr && (a == nullptr || cols != vdim)))
        return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
#define IE_GR_ARGS q, q_ld, a, a_ld, w, w_ld, gates, v, v_ld, state, state_stride, slots, cu_q, out, num_seqs, heads, dim, vdim, cols, q_scale, num_slots, s
#define IE_GR_PICK(SC)                                                        \
    if (dim <= 8) return launch_recurrence<8, 1, SC>(IE_GR_ARGS);             \
    if (dim <= 16) return launch_recurrence<8, 2, SC>(IE_GR_ARGS);            \
    if (dim <= 32) return launch_recurrence<8, 4, SC>(IE_GR_ARGS);            \
    if (dim <= 64) return launch_recurrence<8, 8, SC>(IE_GR_ARGS);            \
    if (dim <= 128) return launch_recurrence<8, 16, SC>(IE_GR_ARGS);          \
    if (dim <= 256) return launch_recurrence<8, 32, SC>(IE_GR_ARGS);          \
    if (dim <= 512) return launch_recurrence<16, 32, SC>(IE_GR_ARGS);
    if (gates != nullptr) { IE_GR_PICK(true) } else { IE_GR_PICK(false) }
#undef IE_GR_PICK
#undef IE_GR_ARGS
    return (int)cudaErrorInvalidValue;  // dim <= 512
}

IE_API int ie_recurrence_readout(const float* o, int cols, const float* gates, const float* weight,
                                 int weight_per_head, float eps, const float* gate_pre, int gate_ld, int gate_silu,
                                 void* out, int out_dtype, long long rows, int heads, int vdim, void* stream) {
    if (rows <= 0) return 0;
    dim3 grid((unsigned)((rows + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16)
        return ie_launch(recurrence_readout_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, o, cols, gates, weight,
                         weight_per_head, eps, gate_pre, gate_ld, gate_silu, (__nv_bfloat16*)out, rows, heads, vdim);
    return ie_launch(recurrence_readout_kernel<float>, grid, dim3(128), 0, s, o, cols, gates, weight,
                     weight_per_head, eps, gate_pre, gate_ld, gate_silu, (float*)out, rows, heads, vdim);
}
