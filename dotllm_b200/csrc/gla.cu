// Gated linear attention: a matrix-valued state per (sequence, head) that decays per key channel.
//
//   alpha_t = sigmoid(z_t)^(1/tau)                      (one decay per key channel, in (0, 1))
//   S_t     = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: [key channels, value channels])
//   o_t     = S_t^T (q_t * q_scale)
//
// followed, in a second kernel, by an RMS norm of every head's o_t over its value channels, a gain
// shared by the heads, and a gate silu(g_t).  State, decays (through log sigmoid, so that a tiny
// sigmoid does not lose its digits before the root is taken), the recurrence and the norm are float32
// whatever the storage type of q, k, v, z and g.
//
// A second form of the same recurrence (z NULL): one constant decay per head, alpha_t = head_decay[h] for every key
// channel and token, with q, k and v passed through silu on their way into the scan:
//   S_t = decay_h S_(t-1) + silu(k_t) silu(v_t)^T,   o_t = S_t^T (silu(q_t) * q_scale)
//
// The scan walks a sequence's new tokens in order, starting from the state that the sequence's slot
// holds and leaving the new state there: a prompt, a part of a prompt and a single decoded token are
// the same loop, so a position's result does not depend on how its sequence was cut into steps.  A
// block owns GLA_COLS value channels of one (sequence, head): columns of S never mix, so blocks need
// nothing from each other.  GLA_SPLIT threads share a column, each holding a run of ROWS
// key channels of it in registers.  Tokens are staged in shared memory a batch at a time (two
// buffers; while a batch is walked the loads of the next one are in flight), rows padded with zeros
// to GLA_SPLIT * ROWS channels so that the walk needs no test and reads its q, k and decays 16 bytes
// at a time.  Per token a thread does its ROWS multiply-adds on the state and on its share of o and
// leaves that share in shared memory; the shares of a batch are summed afterwards, all tokens at
// once, so nothing in the walk waits for another lane.
#include "common.cuh"

#define GLA_COLS 16
#define GLA_SPLIT 16
#define GLA_THREADS (GLA_COLS * GLA_SPLIT)
#define GLA_MAX_DIM 512                  // key channels per head that the scan takes (GLA_SPLIT threads x 32 rows)
#define GLA_STAGE 1024                   // values of q (and of k, and of the decays) staged per batch
#define GLA_MAX_BATCH 16                 // tokens per batch at most

// SINGLE: every sequence of the step brings one token (a decode step).  The same arithmetic in the same order, so the
// same bits; only the staging shrinks to one token, which leaves room for more blocks on a multiprocessor - a decode
// step is thousands of short blocks, each a chain of dependent latencies, and only their number in flight hides those.
template <typename T, int ROWS, bool SINGLE>
__global__ void __launch_bounds__(GLA_THREADS, SINGLE && ROWS <= 8 ? 5 : 1)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int ld,
                const float* __restrict__ z, int z_stride, const float* __restrict__ z_bias,
                const int32_t* __restrict__ cu_new, const int32_t* __restrict__ slots, float* __restrict__ state,
                int n_slots, float* __restrict__ out, int out_stride, int H, int dim, int vdim, float q_scale,
                float inv_tau) {
    constexpr int PAD = GLA_SPLIT * ROWS;                       // staged channels per token, >= dim
    constexpr int BATCH = SINGLE ? 1 : (GLA_STAGE / PAD < GLA_MAX_BATCH ? GLA_STAGE / PAD : GLA_MAX_BATCH);
    constexpr int GLA_LOADS = (BATCH * PAD + GLA_THREADS - 1) / GLA_THREADS;
    constexpr int GLA_VLOADS = (BATCH * GLA_COLS + GLA_THREADS - 1) / GLA_THREADS;
    __shared__ __align__(16) float sq[2][BATCH * PAD], sk[2][BATCH * PAD], sa[2][BATCH * PAD];
    __shared__ float sv[2][GLA_VLOADS * GLA_THREADS];
    __shared__ __align__(16) float sp[BATCH * GLA_COLS * GLA_SPLIT];     // every lane's share of o, per (token, column)
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    // neighbouring lanes hold neighbouring columns: the state's rows are read and written in runs of GLA_COLS values,
    // and a warp reads only two places of the staged q, k and decays at a time
    const int tid = threadIdx.x, r = tid / GLA_COLS, c_local = tid % GLA_COLS;
    const int col0 = blockIdx.x * GLA_COLS;
    const int col = col0 + c_local;
    const bool col_ok = col < vdim;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int slot = slots[b];
    if (slot < 0 || slot >= n_slots || t0 >= t1) return;       // uniform over the block
    float* S = state + ((size_t)slot * H + h) * dim * vdim;
    float s[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
        const int ch = r * ROWS + m;
        s[m] = (ch < dim && col_ok) ? S[(size_t)ch * vdim + col] : 0.f;
    }
    // What a thread fetches for the next batch stays in registers as it was loaded: converting or adding here would
    // make the fetch wait for its own loads, and the walk of the present batch behind it.  Every load is from a valid
    // address (clamped), so that none hides behind a branch; what lies outside the batch is dropped when it is staged.
    T rq[GLA_LOADS], rk[GLA_LOADS], rv[GLA_VLOADS];
    float rz[GLA_LOADS], rb[GLA_LOADS];
    // element e of a batch is (token e / PAD, key channel e % PAD); value e is (token e / GLA_COLS, column e % GLA_COLS)
    auto fetch = [&](int first, int count) {
#pragma unroll
        for (int l = 0; l < GLA_LOADS; ++l) {
            const int e = tid + GLA_THREADS * l;
            const int tok = min(e / PAD, count - 1), ch = min(e % PAD, dim - 1);
            const size_t row = (size_t)(first + tok);
            rq[l] = q[row * ld + h * dim + ch];
            rk[l] = k[row * ld + h * dim + ch];
            rz[l] = z != nullptr ? z[row * z_stride + h * dim + ch] : 0.f;
            rb[l] = z != nullptr ? z_bias[h * dim + ch] : z_bias[h];          // without logits: the head's constant decay
        }
#pragma unroll
        for (int l = 0; l < GLA_VLOADS; ++l) {
            const int e = tid + GLA_THREADS * l;
            const int tok = min(e / GLA_COLS, count - 1), c = min(col0 + e % GLA_COLS, vdim - 1);
            rv[l] = v[(size_t)(first + tok) * ld + h * vdim + c];
        }
    };
    fetch(t0, min(BATCH, t1 - t0));
    int buf = 0;
    for (int first = t0; first < t1; first += BATCH) {
        const int count = min(BATCH, t1 - first);
#pragma unroll
        for (int l = 0; l < GLA_LOADS; ++l) {
            const int e = tid + GLA_THREADS * l;
            if (e < BATCH * PAD) {
                const bool live = e / PAD < count && e % PAD < dim;    // a padded channel decays to nothing and adds nothing
                const float zz = rz[l] + rb[l];
                const float log_sigmoid = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
                float qq = dl_to_f32<T>(rq[l]), kk = dl_to_f32<T>(rk[l]);
                if (z == nullptr) { qq = qq / (1.0f + expf(-qq)); kk = kk / (1.0f + expf(-kk)); }
                sq[buf][e] = live ? qq * q_scale : 0.f;
                sk[buf][e] = live ? kk : 0.f;
                sa[buf][e] = live ? (z != nullptr ? expf(log_sigmoid * inv_tau) : rb[l]) : 0.f;
            }
        }
#pragma unroll
        for (int l = 0; l < GLA_VLOADS; ++l) {
            const float vv = dl_to_f32<T>(rv[l]);
            sv[buf][tid + GLA_THREADS * l] = z != nullptr ? vv : vv / (1.0f + expf(-vv));
        }
        __syncthreads();                                        // the batch is staged; the shares of the batch before are summed
        if (first + BATCH < t1) fetch(first + BATCH, min(BATCH, t1 - first - BATCH));
#pragma unroll 4
        for (int i = 0; i < count; ++i) {                      // tokens depend on each other through s alone: their loads and sums overlap
            const float vt = sv[buf][i * GLA_COLS + c_local];
            const float4* aq = reinterpret_cast<const float4*>(sq[buf] + i * PAD + r * ROWS);
            const float4* ak = reinterpret_cast<const float4*>(sk[buf] + i * PAD + r * ROWS);
            const float4* aa = reinterpret_cast<const float4*>(sa[buf] + i * PAD + r * ROWS);
            float o = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int m = 0; m < ROWS / 4; ++m) {
                const float4 a4 = aa[m], k4 = ak[m], q4 = aq[m];
                s[4 * m] = a4.x * s[4 * m] + k4.x * vt;
                s[4 * m + 1] = a4.y * s[4 * m + 1] + k4.y * vt;
                s[4 * m + 2] = a4.z * s[4 * m + 2] + k4.z * vt;
                s[4 * m + 3] = a4.w * s[4 * m + 3] + k4.w * vt;
                o += s[4 * m] * q4.x;
                o1 += s[4 * m + 1] * q4.y;
                o2 += s[4 * m + 2] * q4.z;
                o3 += s[4 * m + 3] * q4.w;
            }
            sp[(i * GLA_SPLIT + r) * GLA_COLS + c_local] = (o + o1) + (o2 + o3);
        }
        __syncthreads();
        for (int e = tid; e < count * GLA_COLS; e += GLA_THREADS) {
            const float* part = sp + (e / GLA_COLS) * GLA_SPLIT * GLA_COLS + e % GLA_COLS;
            float total = 0.f;
#pragma unroll
            for (int p4 = 0; p4 < GLA_SPLIT; p4 += 4)
                total += (part[p4 * GLA_COLS] + part[(p4 + 1) * GLA_COLS]) + (part[(p4 + 2) * GLA_COLS] + part[(p4 + 3) * GLA_COLS]);
            const int c = col0 + e % GLA_COLS;
            if (c < vdim) out[(size_t)(first + e / GLA_COLS) * out_stride + h * vdim + c] = total;
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

template <typename T>
static int launch_scan(const void* q, const void* k, const void* v, int ld, const float* z, int z_stride, const float* z_bias,
                       const int32_t* cu_new, const int32_t* slots, float* state, int n_slots, float* out, int out_stride,
                       int n_seqs, int H, int dim, int vdim, float q_scale, float inv_tau, bool single, cudaStream_t s) {
    const dim3 grid((vdim + GLA_COLS - 1) / GLA_COLS, H, n_seqs), block(GLA_THREADS);
    const int rows = (dim + GLA_SPLIT - 1) / GLA_SPLIT;
    cudaError_t e;
#define GLA_LAUNCH(R)                                                                                                   \
    if (single)                                                                                                         \
        e = dl_launch_dependent(gla_scan_kernel<T, R, true>, grid, block, 0, s, (const T*)q, (const T*)k, (const T*)v, ld, \
                                z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride, H, dim, vdim, \
                                q_scale, inv_tau);                                                                     \
    else                                                                                                                \
    e = dl_launch_dependent(gla_scan_kernel<T, R, false>, grid, block, 0, s, (const T*)q, (const T*)k, (const T*)v, ld,        \
                            z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride, H, dim, vdim, \
                            q_scale, inv_tau)
    if (rows <= 4) { GLA_LAUNCH(4); }
    else if (rows <= 8) { GLA_LAUNCH(8); }
    else if (rows <= 16) { GLA_LAUNCH(16); }
    else { GLA_LAUNCH(32); }
#undef GLA_LAUNCH
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gla_scan: %s", cudaGetErrorString(e));
    return DL_OK;
}

// q, k [tokens, H*dim] and v [tokens, H*vdim]: views with the common row stride ld (columns of one projection);
// z float32 [tokens, H*dim] (decay logits before the bias), rows z_stride apart; z_bias float32 [H*dim]; with z NULL
// z_bias is float32 [H], one constant decay per head, and q, k, v pass through silu;
// cu_new int32 [n_seqs + 1] (offsets of each sequence's tokens among the step's rows); slots int32 [n_seqs];
// state float32 [n_slots, H, dim, vdim], read and updated; out float32 [n_tokens, H*vdim], rows out_stride apart.
extern "C" int dl_gla_scan(const void* q, const void* k, const void* v, int ld, const float* z, int z_stride,
                           const float* z_bias, int dtype, const int32_t* cu_new, const int32_t* slots, float* state,
                           int n_slots, float* out, int out_stride, int n_seqs, int n_tokens, int H, int dim, int vdim,
                           float q_scale, float tau, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && H > 0 && dim > 0 && vdim > 0 && n_slots > 0, "gla_scan: bad sizes");
    DL_REQUIRE(dim <= GLA_MAX_DIM, "gla_scan: %d key channels per head, the kernel takes up to %d", dim, GLA_MAX_DIM);
    DL_REQUIRE(tau > 0.f, "gla_scan: tau must be positive");
    DL_REQUIRE(out_stride >= H * vdim && (z == nullptr || z_stride >= H * dim), "gla_scan: rows overlap");
    if (n_seqs == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool single = n_tokens == n_seqs;          // no sequence brings less than one token: each brings exactly one
    if (dtype == DL_F32)
        return launch_scan<float>(q, k, v, ld, z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride, n_seqs, H,
                                  dim, vdim, q_scale, 1.0f / tau, single, s);
    if (dtype == DL_BF16)
        return launch_scan<__nv_bfloat16>(q, k, v, ld, z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride,
                                          n_seqs, H, dim, vdim, q_scale, 1.0f / tau, single, s);
    return dl_fail(DL_ERR_UNSUPPORTED, "gla_scan: dtype %d", dtype);
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gain[:] * gate(g[t, h, :]): one warp per (token, head).
// gate_kind 0: silu(g); 1: sigmoid(g).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ g, int g_stride,
                      const float* __restrict__ gain, T* __restrict__ out, int out_stride, int rows, int H, int vdim,
                      float eps, int gate_kind) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long idx = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= (long)rows * H) return;
    const int t = (int)(idx / H), h = (int)(idx % H);
    const float* orow = o + (size_t)t * o_stride + (size_t)h * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += orow[j] * orow[j];
    ss = dl_warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* grow = g + (size_t)t * g_stride + (size_t)h * vdim;
    T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
    for (int j = lane; j < vdim; j += 32) {
        const float gate = dl_to_f32<T>(grow[j]);
        const float sig = 1.0f / (1.0f + expf(-gate));
        dst[j] = dl_from_f32<T>(orow[j] * scale * gain[j] * (gate_kind == 1 ? sig : gate * sig));
    }
}

// The same for heads wider than a warp walks well (a norm over all heads' outputs at once is one head as wide as all): a
// block per (token, head), the row's values waiting in registers across the reduction.
#define HNG_WIDE_THREADS 256
#define HNG_WIDE_MIN 1024
#define HNG_WIDE_PER_THREAD 32           // values a thread keeps: rows of up to 8192 values
template <typename T>
__global__ void __launch_bounds__(HNG_WIDE_THREADS)
head_norm_gate_wide_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ g, int g_stride,
                           const float* __restrict__ gain, T* __restrict__ out, int out_stride, int H, int vdim, float eps,
                           int gate_kind) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t = blockIdx.x / H, h = blockIdx.x % H;
    const float* orow = o + (size_t)t * o_stride + (size_t)h * vdim;
    const T* grow = g + (size_t)t * g_stride + (size_t)h * vdim;
    float v[HNG_WIDE_PER_THREAD], gt[HNG_WIDE_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < HNG_WIDE_PER_THREAD; ++i) {
        const int j = threadIdx.x + i * HNG_WIDE_THREADS;
        v[i] = j < vdim ? orow[j] : 0.f;
        gt[i] = j < vdim ? dl_to_f32<T>(grow[j]) : 0.f;
        ss += v[i] * v[i];
    }
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
    T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
#pragma unroll
    for (int i = 0; i < HNG_WIDE_PER_THREAD; ++i) {
        const int j = threadIdx.x + i * HNG_WIDE_THREADS;
        if (j < vdim) {
            const float sig = 1.0f / (1.0f + expf(-gt[i]));
            dst[j] = dl_from_f32<T>(v[i] * scale * gain[j] * (gate_kind == 1 ? sig : gt[i] * sig));
        }
    }
}

extern "C" int dl_head_norm_gate(const float* o, int o_stride, const void* g, int g_stride, const float* gain, void* out,
                                 int out_stride, int dtype, int rows, int H, int vdim, float eps, int gate_kind, void* stream) {
    DL_REQUIRE(rows >= 0 && H > 0 && vdim > 0 && eps > 0.f, "head_norm_gate: bad arguments");
    DL_REQUIRE(gate_kind == 0 || gate_kind == 1, "head_norm_gate: gate kind %d (0: silu, 1: sigmoid)", gate_kind);
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long warps = (long)rows * H;
    const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
    cudaError_t e;
    if (vdim >= HNG_WIDE_MIN && vdim <= HNG_WIDE_THREADS * HNG_WIDE_PER_THREAD && (dtype == DL_F32 || dtype == DL_BF16)) {
        const dim3 wide((unsigned)warps), threads(HNG_WIDE_THREADS);
        if (dtype == DL_F32)
            e = dl_launch_dependent(head_norm_gate_wide_kernel<float>, wide, threads, 0, s, o, o_stride, (const float*)g, g_stride, gain,
                                    (float*)out, out_stride, H, vdim, eps, gate_kind);
        else
            e = dl_launch_dependent(head_norm_gate_wide_kernel<__nv_bfloat16>, wide, threads, 0, s, o, o_stride, (const __nv_bfloat16*)g,
                                    g_stride, gain, (__nv_bfloat16*)out, out_stride, H, vdim, eps, gate_kind);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "head_norm_gate: %s", cudaGetErrorString(e));
        return DL_OK;
    }
    if (dtype == DL_F32)
        e = dl_launch_dependent(head_norm_gate_kernel<float>, grid, block, 0, s, o, o_stride, (const float*)g, g_stride, gain,
                                (float*)out, out_stride, rows, H, vdim, eps, gate_kind);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, s, o, o_stride, (const __nv_bfloat16*)g,
                                g_stride, gain, (__nv_bfloat16*)out, out_stride, rows, H, vdim, eps, gate_kind);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "head_norm_gate: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "head_norm_gate: %s", cudaGetErrorString(e));
    return DL_OK;
}
