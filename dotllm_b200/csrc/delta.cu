// The gated delta rule with a decay per key channel: a matrix-valued state per (sequence, head) that is
// decayed row by row, corrected towards the token's value along the token's key, and read by the query.
//
//   S <- diag(g_t) S                      (S: [key channels, value channels]; g_t in (0, 1) per key channel)
//   u  = beta_t (v_t - S^T k_t)           (what the state gets wrong about v_t along k_t, times a step size)
//   S <- S + k_t u^T
//   o_t = S^T q_t                          (after the write: the token reads what it wrote)
//
// In front of it, a short causal convolution over time per channel of q, k and v (taps [channels, K], the last
// column meets the current token, zeros before the sequence's start), silu, unit length per head for q and k
// (x / sqrt(sum x^2 + unit_eps), q also times q_scale), the step size beta = sigmoid(b) and the decay
// g = exp(-exp(A_h) softplus(z + dt)).  All of that is one kernel over tokens (`delta_prepare`), float32 from
// the convolution's sum on; the recurrence is a second kernel (`delta_scan`), float32 throughout.
//
// What a sequence carries from step to step lies in one float32 vector per slot: the state S of every head
// [H, dim, vdim], and behind it the convolution's last K - 1 inputs [K - 1, channels] (oldest first).  A prompt, a
// part of a prompt and one decoded token are the same code, so a position's result does not depend on how the
// sequence was cut into steps.
//
// The scan: columns of S never mix, so a block owns DR_COLS value channels of one (sequence, head).  DR_SPLIT
// lanes of one warp share a column, each with a run of ROWS key channels in registers; per token they take the
// partial sums of S^T (g k), exchange them by shuffles inside the warp (no block barrier per token), write the decayed
// rows plus the correction, and read the new rows with q.  Tokens are staged in shared memory a batch at a time from
// registers that were loaded while the batch before was walked.
#include "common.cuh"

#define DP_THREADS 128
#define DP_RUN 16                                          // tokens a block walks in a row, at most
#define DP_MAX_TAPS 64                                     // taps of the short convolution a thread keeps in registers

__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One block per (run of tokens, part): the parts are the G query heads, the G key heads and the H value heads of a token, so
// that a step of few tokens still fills the machine; a step of many tokens gives a block `per_block` of them in a row.
// x: the stacked projection's rows (q channels, then k, then v: C = 2*G*dim + H*vdim columns from column 0 of `x`, rows
// `ld` apart); taps [C, K] of x's type; history: float32 [K - 1, C] per slot at `hist` + slot * slot_stride.  Row t is
// token (t - cu_new[b]) of sequence b = token_seq[t].  A value head's block also writes its head's decays and step size.
// A thread keeps its channel's taps and last inputs in registers (KMAX >= K places, the current token's last, zeros in
// front), moves them on by one place per token, and fills them anew where the run enters another sequence.
template <typename T, int KMAX>
__global__ void __launch_bounds__(DP_THREADS)
delta_prepare_kernel(const T* __restrict__ x, int ld, const T* __restrict__ taps, int K, float* __restrict__ hist, long slot_stride,
                     int n_slots, const int32_t* __restrict__ token_seq, const int32_t* __restrict__ cu_new,
                     const int32_t* __restrict__ slots, const T* __restrict__ b_logit, int b_stride,
                     const float* __restrict__ z, int z_stride, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, float* __restrict__ qo, float* __restrict__ ko, float* __restrict__ vo,
                     float* __restrict__ go, float* __restrict__ bo, int H, int G, int dim, int vdim, float q_scale,
                     float unit_eps, int update_history, int n_tokens, int per_block, int head_decay) {
    extern __shared__ float dp_y[];                       // [per_block, dim]: a query or key head's channels after convolution and silu
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int part = blockIdx.y;
    const int qk = 2 * G * dim, C = qk + H * vdim;
    const bool is_v = part >= 2 * G;
    const int c0 = is_v ? qk + (part - 2 * G) * vdim : part * dim, width = is_v ? vdim : dim;
    const int t_begin = blockIdx.x * per_block, t_end = min(n_tokens, t_begin + per_block);
    __shared__ int dp_seq[DP_RUN], dp_slot[DP_RUN], dp_place[DP_RUN];   // per token of the run; a slot outside the memory reads -1
    if (threadIdx.x < t_end - t_begin) {
        const int b = token_seq[t_begin + threadIdx.x], slot = slots[b];
        dp_seq[threadIdx.x] = b;
        dp_slot[threadIdx.x] = slot >= 0 && slot < n_slots ? slot : -1;
        dp_place[threadIdx.x] = t_begin + threadIdx.x - cu_new[b];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < width; d += DP_THREADS) {
        const int c = c0 + d;
        float tap[KMAX], in[KMAX];
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {                  // place KMAX - 1 - lag meets the input `lag` tokens back
            const int lag = KMAX - 1 - i;
            tap[i] = lag < K ? dl_to_f32<T>(taps[(size_t)c * K + (K - 1 - lag)]) : 0.f;
            in[i] = 0.f;
        }
        int before = -1;
        float ahead = dl_to_f32<T>(x[(size_t)t_begin * ld + c]);
        for (int t = t_begin; t < t_end; ++t) {
            const float now = ahead;                      // the next token's input is under way while this one is worked on
            if (t + 1 < t_end) ahead = dl_to_f32<T>(x[(size_t)(t + 1) * ld + c]);
            const int b = dp_seq[t - t_begin], slot = dp_slot[t - t_begin];
            if (slot < 0) { before = -1; continue; }
            const int j = dp_place[t - t_begin];          // the token's place among its sequence's new tokens
            float* hs = hist + (size_t)slot * slot_stride;
            if (b != before) {
                // new rows hold the last j inputs; older ones lie in the history, whose row K - 2 is the newest
#pragma unroll
                for (int lag = 1; lag < KMAX; ++lag)
                    if (lag < K)
                        in[KMAX - 1 - lag] = lag <= j ? dl_to_f32<T>(x[(size_t)(t - lag) * ld + c])
                                                      : hs[(size_t)(K - 1 - (lag - j)) * C + c];
                before = b;
            }
            in[KMAX - 1] = now;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < KMAX; ++i) acc = fmaf(tap[i], in[i], acc);          // oldest first; a place in front of the taps adds 0 * 0
#pragma unroll
            for (int i = 0; i + 1 < KMAX; ++i) in[i] = in[i + 1];
            const float y = acc / (1.0f + expf(-acc));
            if (is_v) vo[(size_t)t * H * vdim + (c - qk)] = y;
            else dp_y[(t - t_begin) * dim + d] = y;
            if (update_history) {
                // a step of one token a sequence: this thread is the only reader of the channel's history and moves it on itself
                for (int i = 0; i + 1 < K - 1; ++i) hs[(size_t)i * C + c] = hs[(size_t)(i + 1) * C + c];
                if (K > 1) hs[(size_t)(K - 2) * C + c] = now;
            }
        }
    }
    if (is_v) {
        const int h = part - 2 * G;
        const float rate = expf(a_log[h]);
        const int items = (t_end - t_begin) * dim;         // (token, key channel) pairs, four loads of a thread under way
        for (int first = threadIdx.x; first < items; first += 4 * DP_THREADS) {
            float zs[4];
            int at[4], ch[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = first + u * DP_THREADS;
                at[u] = t_begin + idx / dim, ch[u] = h * dim + idx % dim;
                zs[u] = idx < items ? z[(size_t)at[u] * z_stride + (head_decay ? h : ch[u])] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (first + u * DP_THREADS >= items) break;
                if (dp_slot[at[u] - t_begin] < 0) continue;
                go[(size_t)at[u] * H * dim + ch[u]] = expf(-rate * dr_softplus(zs[u] + dt_bias[head_decay ? h : ch[u]]));
            }
        }
        for (int t = t_begin + threadIdx.x; t < t_end; t += DP_THREADS) {
            if (dp_slot[t - t_begin] < 0) continue;
            bo[(size_t)t * H + h] = 1.0f / (1.0f + expf(-dl_to_f32<T>(b_logit[(size_t)t * b_stride + h])));
        }
        return;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    for (int t = t_begin + (threadIdx.x >> 5); t < t_end; t += DP_THREADS / 32) {  // a warp per token
        if (dp_slot[t - t_begin] < 0) continue;
        const float* y = dp_y + (t - t_begin) * dim;
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) ss += y[d] * y[d];
        ss = dl_warp_sum(ss);
        const float r = (1.0f / sqrtf(ss + unit_eps)) * (part < G ? q_scale : 1.0f);
        float* dst = part < G ? qo + (size_t)t * G * dim + (size_t)part * dim : ko + (size_t)t * G * dim + (size_t)(part - G) * dim;
        for (int d = lane; d < dim; d += 32) dst[d] = y[d] * r;
    }
}

// The history after a step of any shape: the last K - 1 inputs of each sequence, oldest first.  One thread per (sequence,
// channel); runs behind delta_prepare (which read the old history).
template <typename T>
__global__ void __launch_bounds__(DP_THREADS)
delta_history_kernel(const T* __restrict__ x, int ld, int K, float* __restrict__ hist, long slot_stride, int n_slots,
                     const int32_t* __restrict__ cu_new, const int32_t* __restrict__ slots, int C) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int b = blockIdx.x;
    const int slot = slots[b];
    const int t0 = cu_new[b], n = cu_new[b + 1] - t0;
    if (slot < 0 || slot >= n_slots || n <= 0) return;
    float* hs = hist + (size_t)slot * slot_stride;
    const int keep = K - 1;
    const int c = blockIdx.y * DP_THREADS + threadIdx.x;
    if (c >= C) return;
    for (int i = 0; i < keep; ++i) {                      // ascending: a place is read (at i + n) before it is written
        const int src = i + n;                            // index in (old history ++ new inputs)
        hs[(size_t)i * C + c] = src < keep ? hs[(size_t)src * C + c] : dl_to_f32<T>(x[(size_t)(t0 + src - keep) * ld + c]);
    }
}

#define DR_SPLIT 8                                        // lanes that share a column
#define DR_WARPS 4
#define DR_COLS (DR_WARPS * 32 / DR_SPLIT)               // value channels per block
#define DR_THREADS (DR_WARPS * 32)
#define DR_MAX_DIM 512
#define DR_STAGE 1024                                     // key channels of q (and of k, and of the decays) staged per batch
#define DR_MAX_BATCH 16

template <int ROWS, bool SINGLE>
__global__ void __launch_bounds__(DR_THREADS)
delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, const int32_t* __restrict__ cu_new,
                  const int32_t* __restrict__ slots, float* __restrict__ state, long slot_stride, int n_slots,
                  float* __restrict__ out, int H, int G, int dim, int vdim) {
    constexpr int PAD = DR_SPLIT * ROWS;                  // staged channels per token, >= dim
    constexpr int RUN = ROWS + 4;                         // a lane's run of channels, shifted so that the lanes' 16-byte reads miss each other's banks
    constexpr int ROW = DR_SPLIT * RUN;
    constexpr int BATCH = SINGLE ? 1 : (DR_STAGE / PAD < DR_MAX_BATCH ? (DR_STAGE / PAD < 1 ? 1 : DR_STAGE / PAD) : DR_MAX_BATCH);
    constexpr int LOADS = (BATCH * PAD + DR_THREADS - 1) / DR_THREADS;
    constexpr int VLOADS = (BATCH * DR_COLS + DR_THREADS - 1) / DR_THREADS;
    __shared__ __align__(16) float sq[2][BATCH * ROW], sk[2][BATCH * ROW], sg[2][BATCH * ROW];
    __shared__ float sv[2][VLOADS * DR_THREADS], sb[2][BATCH];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int b = blockIdx.z, h = blockIdx.y, kvh = h / (H / G);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane % DR_SPLIT, c_local = warp * (32 / DR_SPLIT) + lane / DR_SPLIT;
    const int col0 = blockIdx.x * DR_COLS, col = col0 + c_local;
    const bool col_ok = col < vdim;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int slot = slots[b];
    if (slot < 0 || slot >= n_slots || t0 >= t1) return;  // uniform over the block
    float* S = state + (size_t)slot * slot_stride + (size_t)h * dim * vdim;
    float s[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
        const int ch = r * ROWS + m;
        s[m] = (ch < dim && col_ok) ? S[(size_t)ch * vdim + col] : 0.f;
    }
    float rq[LOADS], rk[LOADS], rg[LOADS], rv[VLOADS], rb = 0.f;
    auto fetch = [&](int first, int count) {              // every load from a valid (clamped) address; what lies outside is dropped when staged
#pragma unroll
        for (int l = 0; l < LOADS; ++l) {
            const int e = tid + DR_THREADS * l;
            const int tok = min(e / PAD, count - 1), ch = min(e % PAD, dim - 1);
            const size_t row = (size_t)(first + tok);
            rq[l] = q[row * G * dim + kvh * dim + ch];
            rk[l] = k[row * G * dim + kvh * dim + ch];
            rg[l] = g[row * H * dim + h * dim + ch];
        }
#pragma unroll
        for (int l = 0; l < VLOADS; ++l) {
            const int e = tid + DR_THREADS * l;
            const int tok = min(e / DR_COLS, count - 1), c = min(col0 + e % DR_COLS, vdim - 1);
            rv[l] = v[(size_t)(first + tok) * H * vdim + h * vdim + c];
        }
        rb = beta[(size_t)(first + min(tid, count - 1)) * H + h];
    };
    fetch(t0, min(BATCH, t1 - t0));
    int buf = 0;
    for (int first = t0; first < t1; first += BATCH) {
        const int count = min(BATCH, t1 - first);
#pragma unroll
        for (int l = 0; l < LOADS; ++l) {
            const int e = tid + DR_THREADS * l;
            if (e < BATCH * PAD) {
                const int tok = e / PAD, ch = e % PAD;
                const bool live = tok < count && ch < dim;       // a padded channel holds zeros and stays zero
                const int at = tok * ROW + (ch / ROWS) * RUN + ch % ROWS;
                sq[buf][at] = live ? rq[l] : 0.f;
                sk[buf][at] = live ? rk[l] : 0.f;
                sg[buf][at] = live ? rg[l] : 0.f;
            }
        }
#pragma unroll
        for (int l = 0; l < VLOADS; ++l) sv[buf][tid + DR_THREADS * l] = rv[l];
        if (tid < BATCH) sb[buf][tid] = rb;
        __syncthreads();                                  // the batch is staged (and every lane is done with the other buffer's batch before it is refilled)
        if (first + BATCH < t1) fetch(first + BATCH, min(BATCH, t1 - first - BATCH));
        // The operands of a token are read into registers while the token before it is walked.  Between two states lie only
        // the dot product with g k, its shuffles, the step and one multiply-add: (g S)^T k = S^T (g k), and S' = g S + k u^T.
        // The read-out o = S'^T q hangs on the new state but nothing hangs on it, so its sums and shuffles run beside the
        // next token's chain.
        float4 nq[ROWS / 4], nk[ROWS / 4], ng[ROWS / 4];
        float nv, nb;
        auto operands = [&](int i) {
            const float4* aq = reinterpret_cast<const float4*>(sq[buf] + i * ROW + r * RUN);
            const float4* ak = reinterpret_cast<const float4*>(sk[buf] + i * ROW + r * RUN);
            const float4* ag = reinterpret_cast<const float4*>(sg[buf] + i * ROW + r * RUN);
#pragma unroll
            for (int m = 0; m < ROWS / 4; ++m) nq[m] = aq[m], nk[m] = ak[m], ng[m] = ag[m];
            nv = sv[buf][i * DR_COLS + c_local];
            nb = sb[buf][i];
        };
        constexpr bool AHEAD = ROWS <= 16;                // wider runs leave no registers for a second set of operands
        if (AHEAD) operands(0);
        float* o_at = out + (size_t)first * H * vdim + h * vdim + col;
#pragma unroll(AHEAD ? 2 : 1)
        for (int i = 0; i < count; ++i, o_at += (size_t)H * vdim) {
            if (!AHEAD) operands(i);
            float kk[ROWS], gg[ROWS], qq[ROWS];
            const float vt = nv, bt = nb;
#pragma unroll
            for (int m = 0; m < ROWS / 4; ++m) {
                const float4 g4 = ng[m], k4 = nk[m], q4 = nq[m];
                kk[4 * m] = k4.x, kk[4 * m + 1] = k4.y, kk[4 * m + 2] = k4.z, kk[4 * m + 3] = k4.w;
                gg[4 * m] = g4.x, gg[4 * m + 1] = g4.y, gg[4 * m + 2] = g4.z, gg[4 * m + 3] = g4.w;
                qq[4 * m] = q4.x, qq[4 * m + 1] = q4.y, qq[4 * m + 2] = q4.z, qq[4 * m + 3] = q4.w;
            }
            if (AHEAD) operands(min(i + 1, BATCH - 1));   // the next token's (the batch's last reads a staged place again)
            float pk[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < ROWS; ++m) pk[m & 3] = fmaf(s[m], gg[m] * kk[m], pk[m & 3]);
            float sk_ = (pk[0] + pk[1]) + (pk[2] + pk[3]);
#pragma unroll
            for (int m = 0; m < ROWS; ++m) s[m] *= gg[m];
#pragma unroll
            for (int o = DR_SPLIT / 2; o > 0; o >>= 1) sk_ += __shfl_xor_sync(0xffffffffu, sk_, o);
            const float u = bt * (vt - sk_);
            float pq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < ROWS; ++m) {
                s[m] = fmaf(kk[m], u, s[m]);
                pq[m & 3] = fmaf(s[m], qq[m], pq[m & 3]);
            }
            float sq_ = (pq[0] + pq[1]) + (pq[2] + pq[3]);
#pragma unroll
            for (int o = DR_SPLIT / 2; o > 0; o >>= 1) sq_ += __shfl_xor_sync(0xffffffffu, sq_, o);
            if (r == 0 && col_ok) *o_at = sq_;
        }
        buf ^= 1;
    }
    if (col_ok) {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
            const int ch = r * ROWS + m;
            if (ch < dim) S[(size_t)ch * vdim + col] = s[m];
        }
    }
}

// x [tokens, >= C] of `dtype` (rows ld apart): q channels [G*dim], k channels [G*dim], v channels [H*vdim]; taps [C, K] of
// `dtype`; b_logit [tokens, H] of `dtype` (rows b_stride apart); z float32 [tokens, H*dim] (rows z_stride apart);
// dt_bias float32 [H*dim] (with `head_decay`: z [tokens, H] and dt_bias [H], one decay for all key channels of a head);
// a_log float32 [H]; slot memory float32: S at `state`, the history at `hist`, both
// slot_stride floats a slot.  Outputs float32, contiguous: q, k [tokens, G*dim], v, o [tokens, H*vdim], g [tokens, H*dim],
// beta [tokens, H].
extern "C" int dl_delta_rule(const void* x, int ld, const void* taps, int K, int dtype, const void* b_logit, int b_stride,
                             const float* z, int z_stride, const float* dt_bias, const float* a_log,
                             const int32_t* token_seq, const int32_t* cu_new, const int32_t* slots, float* state, float* hist,
                             long slot_stride, int n_slots, float* qo, float* ko, float* vo, float* go, float* bo, float* out,
                             int n_seqs, int n_tokens, int H, int G, int dim, int vdim, float q_scale, float unit_eps,
                             int head_decay, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && n_tokens >= 0 && H > 0 && G > 0 && dim > 0 && vdim > 0 && n_slots > 0 && K >= 1, "delta_rule: bad sizes");
    DL_REQUIRE(H % G == 0, "delta_rule: %d heads are not a multiple of %d key heads", H, G);
    DL_REQUIRE(K <= DP_MAX_TAPS, "delta_rule: a convolution of %d taps, the kernel takes up to %d", K, DP_MAX_TAPS);
    DL_REQUIRE(dim <= DR_MAX_DIM, "delta_rule: %d key channels per head, the kernel takes up to %d", dim, DR_MAX_DIM);
    const int C = 2 * G * dim + H * vdim;
    DL_REQUIRE(ld >= C && z_stride >= (head_decay ? H : H * dim) && b_stride >= H, "delta_rule: rows overlap");
    DL_REQUIRE(dtype == DL_F32 || dtype == DL_BF16, "delta_rule: dtype %d", dtype);
    if (n_seqs == 0 || n_tokens == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool single = n_tokens == n_seqs;               // every sequence brings exactly one token
    // enough blocks for a few rounds over the machine; beyond that a block walks a run of tokens
    const long rounds = (long)n_tokens * (2 * G + H) / 4096;
    const int per_block = rounds < 1 ? 1 : rounds > DP_RUN ? DP_RUN : (int)rounds;
    const size_t smem = (size_t)per_block * dim * sizeof(float);
    cudaError_t e;
    const dim3 pgrid((n_tokens + per_block - 1) / per_block, 2 * G + H);
#define DP_LAUNCH(T, KMAX)                                                                                                    \
    e = dl_launch_dependent(delta_prepare_kernel<T, KMAX>, pgrid, dim3(DP_THREADS), smem, s, (const T*)x, ld, (const T*)taps, \
                            K, hist, slot_stride, n_slots, token_seq, cu_new, slots, (const T*)b_logit, b_stride, z,          \
                            z_stride, dt_bias, a_log, qo, ko, vo, go, bo, H, G, dim, vdim, q_scale, unit_eps,                 \
                            single ? 1 : 0, n_tokens, per_block, head_decay)
    if (dtype == DL_F32) {
        if (K <= 4) { DP_LAUNCH(float, 4); } else if (K <= 8) { DP_LAUNCH(float, 8); } else if (K <= 16) { DP_LAUNCH(float, 16); } else { DP_LAUNCH(float, DP_MAX_TAPS); }
    } else {
        if (K <= 4) { DP_LAUNCH(__nv_bfloat16, 4); } else if (K <= 8) { DP_LAUNCH(__nv_bfloat16, 8); } else if (K <= 16) { DP_LAUNCH(__nv_bfloat16, 16); }
        else { DP_LAUNCH(__nv_bfloat16, DP_MAX_TAPS); }
    }
#undef DP_LAUNCH
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "delta_prepare: %s", cudaGetErrorString(e));
    if (!single && K > 1) {
        if (dtype == DL_F32)
            e = dl_launch_dependent(delta_history_kernel<float>, dim3(n_seqs, (C + DP_THREADS - 1) / DP_THREADS), dim3(DP_THREADS), 0, s, (const float*)x, ld, K, hist,
                                    slot_stride, n_slots, cu_new, slots, C);
        else
            e = dl_launch_dependent(delta_history_kernel<__nv_bfloat16>, dim3(n_seqs, (C + DP_THREADS - 1) / DP_THREADS), dim3(DP_THREADS), 0, s,
                                    (const __nv_bfloat16*)x, ld, K, hist, slot_stride, n_slots, cu_new, slots, C);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "delta_history: %s", cudaGetErrorString(e));
    }
    const dim3 grid((vdim + DR_COLS - 1) / DR_COLS, H, n_seqs), block(DR_THREADS);
    const int rows = (dim + DR_SPLIT - 1) / DR_SPLIT;
    // few blocks that walk a long run of tokens want a multiprocessor each: they start when the kernels before have ended
    const bool early = (long)grid.x * grid.y * grid.z > 2L * dl_sm_count();
#define DR_LAUNCH(R)                                                                                                          \
    if (single)                                                                                                               \
        e = dl_launch_dependent_if(early, delta_scan_kernel<R, true>, grid, block, 0, s, (const float*)qo, (const float*)ko,            \
                                (const float*)vo, (const float*)go, (const float*)bo, cu_new, slots, state, slot_stride,      \
                                n_slots, out, H, G, dim, vdim);                                                               \
    else                                                                                                                      \
        e = dl_launch_dependent_if(early, delta_scan_kernel<R, false>, grid, block, 0, s, (const float*)qo, (const float*)ko,           \
                                (const float*)vo, (const float*)go, (const float*)bo, cu_new, slots, state, slot_stride,      \
                                n_slots, out, H, G, dim, vdim)
    if (rows <= 4) { DR_LAUNCH(4); }
    else if (rows <= 8) { DR_LAUNCH(8); }
    else if (rows <= 16) { DR_LAUNCH(16); }
    else if (rows <= 32) { DR_LAUNCH(32); }
    else { DR_LAUNCH(64); }
#undef DR_LAUNCH
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "delta_scan: %s", cudaGetErrorString(e));
    return DL_OK;
}
