// A feed-forward of many small experts of which every token uses a few.
//
//   router:  z = R x + b (float32);  the `top` largest z choose the experts, ties to the lower index;
//            their weights are the softmax over the chosen z alone (scoring 0), or sigmoid(z) of each
//            chosen expert as it is, not renormalised (scoring 1), or the chosen experts' shares s of the softmax
//            over ALL experts (scoring 2), optionally chosen by s + a correction per expert, divided by their sum
//            (+ 1e-20) and multiplied by a constant
//   identity experts: the experts behind the last one with matrices give back their input, y = x
//   expert:  y = D_e act(G_e x, U_e x)       (act: one of the gatings of gating.cuh), or D_e act(U_e x)
//            for an activation of one product; the weight multiplies y, or (a row scale) the expert's input x
//   output:  sum over the chosen experts of weight * y   (+ an addend per token, e.g. a shared expert,
//            which a per-token logit may gate: addend * sigmoid(logit))
//
// Kernels, none of which needs the host to know which experts were chosen (a step can be captured in
// a graph): the choice (a warp per token, from the float32 logits of the router's product), the gated product (a block per (token, chosen
// expert) row, a warp per output: the row's activations wait in shared memory as float32 and every
// lane walks its share of the expert's weight row), and the down product with the weighted sum in
// it (a block per token).  Every output is one warp's sum in an order that depends only on the sizes,
// so a token's result does not depend on what else is in the step.
#include "common.cuh"
#include "gating.cuh"

#define EX_WARPS 8
#define EX_OUT_PER_BLOCK 64

// logits float32 [rows, E] (the router's product), bias float32 [E] or NULL.  A warp per row.
// scoring 2: the weights are the chosen experts' shares of the softmax over ALL experts, not renormalised.  With
// `groups` > 0 the experts lie in that many equal runs of neighbours; a run's score is its largest logit, and only the
// experts of the `keep_groups` best runs (ties to the lower index) can be chosen.  `correction` (float32 [E] or NULL, scoring 2
// without groups): the choice goes by share + correction, the weights stay the shares.  `normalise`: the chosen weights are
// divided by their sum + 1e-20.  Every weight is multiplied by `weight_scale`.
__global__ void __launch_bounds__(32 * EX_WARPS)
route_topk_kernel(const float* __restrict__ z, int z_stride, const float* __restrict__ bias, int32_t* __restrict__ ids,
                  float* __restrict__ weights, int rows, int E, int top, int scoring, int groups, int keep_groups,
                  const float* __restrict__ correction, int normalise, float weight_scale) {
    extern __shared__ float route_smem[];            // per warp: E logits, `top` chosen values, `groups` run scores, E shares
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * EX_WARPS + warp;
    if (row >= rows) return;                          // warps are independent below
    float* logits = route_smem + (size_t)warp * (E + top + groups + (correction != nullptr ? E : 0));
    float* chosen = logits + E;
    float* run_best = chosen + top;
    float* shares = run_best + groups;                // [E], only with a correction
    float all_max = -INFINITY, all_sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        logits[e] = z[(size_t)row * z_stride + e] + (bias != nullptr ? bias[e] : 0.f);
        all_max = fmaxf(all_max, logits[e]);
    }
    __syncwarp();
    if (scoring == 2) {                               // the softmax's denominator over every expert, before any is ruled out
        all_max = dl_warp_max(all_max);
        for (int e = lane; e < E; e += 32) all_sum += expf(logits[e] - all_max);
        all_sum = dl_warp_sum(all_sum);
        if (correction != nullptr) {                  // the choice goes by share + correction: the logits' places hold that sum
            for (int e = lane; e < E; e += 32) {
                shares[e] = expf(logits[e] - all_max) / all_sum;
                logits[e] = shares[e] + correction[e];
            }
            __syncwarp();
        }
    }
    if (groups > 0 && keep_groups < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, logits[e]);
            run_best[g] = best;
        }
        __syncwarp();
        for (int j = 0; j < keep_groups; ++j) {       // mark the best runs by +inf in their score's place
            float best = -INFINITY;
            int at = groups;
            for (int g = lane; g < groups; g += 32) {
                const float v = run_best[g];
                if (v != INFINITY && (at == groups || v > best)) { best = v; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa < groups && (at == groups || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0 && at < groups) run_best[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (run_best[e / per] != INFINITY) logits[e] = -INFINITY;
        __syncwarp();
    }
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32) {
            const float v = logits[e];
            if (at == E || v > best) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa < E && (at == E || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
        }
        if (lane == 0) {
            ids[(size_t)row * top + j] = at < E ? at : 0;
            chosen[j] = best;
            if (at < E) logits[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        if (scoring == 1) {                           // each chosen expert's own sigmoid (monotone in z: the same choice)
            for (int j = 0; j < top; ++j) weights[(size_t)row * top + j] = 1.0f / (1.0f + expf(-chosen[j]));
            return;
        }
        if (scoring == 2) {
            float sum = 0.f;
            for (int j = 0; j < top; ++j) {
                const int at = ids[(size_t)row * top + j];
                chosen[j] = correction != nullptr ? shares[at] : expf(chosen[j] - all_max) / all_sum;
                sum += chosen[j];
            }
            const float f = normalise ? weight_scale / (sum + 1e-20f) : weight_scale;
            for (int j = 0; j < top; ++j) weights[(size_t)row * top + j] = chosen[j] * f;
            return;
        }
        const float m = chosen[0];
        float sum = 0.f;
        for (int j = 0; j < top; ++j) sum += expf(chosen[j] - m);
        for (int j = 0; j < top; ++j) weights[(size_t)row * top + j] = expf(chosen[j] - m) / sum;
    }
}

// z float32 [rows, E], rows z_stride apart; bias float32 [E] or NULL; ids int32 [rows, top]; weights float32 [rows, top].
extern "C" int dl_route_topk(const float* z, int z_stride, const float* bias, int32_t* ids, float* weights, int rows, int E,
                             int top, int scoring, int groups, int keep_groups, const float* correction, int normalise,
                             float weight_scale, void* stream) {
    DL_REQUIRE(rows >= 0 && E > 0 && top > 0 && top <= E && z_stride >= E, "route_topk: bad sizes E=%d top=%d", E, top);
    DL_REQUIRE(scoring >= 0 && scoring <= 2, "route_topk: scoring %d (0: softmax over the chosen, 1: sigmoid, 2: softmax over all)", scoring);
    DL_REQUIRE(groups >= 0 && (groups == 0 || (E % groups == 0 && keep_groups > 0 && keep_groups <= groups &&
                                               top <= keep_groups * (E / groups))),
               "route_topk: %d experts in %d runs of which %d stay cannot give %d choices", E, groups, keep_groups, top);
    DL_REQUIRE((correction == nullptr && !normalise && weight_scale == 1.0f) || (scoring == 2 && groups == 0),
               "route_topk: a correction, normalised weights and a scale go with the softmax over all experts, without groups");
    const size_t smem = (size_t)EX_WARPS * (E + top + groups + (correction != nullptr ? E : 0)) * sizeof(float);
    DL_REQUIRE(smem <= 48 * 1024, "route_topk: %d experts are more than the kernel's shared memory takes", E);
    if (rows == 0) return DL_OK;
    const dim3 grid((rows + EX_WARPS - 1) / EX_WARPS), block(32 * EX_WARPS);
    cudaError_t e = dl_launch_dependent(route_topk_kernel, grid, block, smem, (cudaStream_t)stream, z, z_stride, bias, ids, weights,
                                        rows, E, top, scoring, groups, keep_groups, correction, normalise, weight_scale);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "route_topk: %s", cudaGetErrorString(e));
    return DL_OK;
}

// A warp's dot product of a weight row with activations that wait in shared memory as float32.  With `vec` every
// lane takes 16 bytes of the row at a time (the caller has checked the rows' width and address), and the activations
// lie permuted so that the values the 32 lanes need at one time fall into 32 different banks: within each run of
// 32 * N values, value c sits at (c % N) * 32 + c / N (N values a lane, ex_place).  Without `vec`, as they come.
template <typename T> struct ExVec;
template <> struct ExVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ float dot(const float* w, const float* x) {
        const float4 a = *reinterpret_cast<const float4*>(w);
        return a.x * x[0] + a.y * x[32] + a.z * x[64] + a.w * x[96];
    }
};
template <> struct ExVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ float dot(const __nv_bfloat16* w, const float* x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(w);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc += __low2float(p[i]) * x[64 * i] + __high2float(p[i]) * x[64 * i + 32];
        return acc;
    }
};

template <typename T>
__device__ __forceinline__ int ex_place(int c, bool vec) {
    constexpr int N = ExVec<T>::N, RUN = 32 * ExVec<T>::N;
    return vec ? (c / RUN) * RUN + (c % N) * 32 + (c % RUN) / N : c;
}
// Outputs a block computes for its row: EX_OUT_PER_BLOCK, halved (down to one per warp) while the launch would leave
// multiprocessors without a block - a decode step has few rows, and each streams whole matrices.
static inline int ex_outputs_per_block(int rows, int outputs) {
    int per_block = EX_OUT_PER_BLOCK;
    while (per_block > EX_WARPS && (long long)rows * ((outputs + per_block - 1) / per_block) < 4 * 148) per_block /= 2;
    return per_block;
}

// floats of shared memory that K staged activations take (whole runs when permuted)
static inline size_t ex_staged(int K, int n_per_lane) { return (size_t)((K + 32 * n_per_lane - 1) / (32 * n_per_lane)) * 32 * n_per_lane; }

template <typename T>
__device__ __forceinline__ float ex_row_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane, bool vec) {
    float acc = 0.f;
    if (vec) {
        constexpr int N = ExVec<T>::N;
        for (int c = lane * N; c < K; c += 32 * N) acc += ExVec<T>::dot(w + c, x + (c - lane * N) + lane);
    } else {
        for (int c = lane; c < K; c += 32) acc += x[c] * dl_to_f32<T>(w[c]);
    }
    return dl_warp_sum(acc);
}

// Row r = (token r / top, chosen expert ids[r]):  out[r, n] = act(G_e[n, :] . x[token], U_e[n, :] . x[token]).
// w: [E, 2 * ff, K], an expert's gate rows first, then its up rows; for an activation of one product w is [E, ff, K]
// and out[r, n] = act(U_e[n, :] . x[token]).  With `row_scale` (float32 [rows]) the row's input is x[token] * row_scale[r].
template <typename T>
__global__ void __launch_bounds__(32 * EX_WARPS)
expert_gate_up_kernel(const T* __restrict__ x, int x_stride, const int32_t* __restrict__ ids, const T* __restrict__ w,
                      T* __restrict__ out, int top, int K, int ff, int E, int kind, float limit, float alpha, int vec, int per_block,
                      const float* __restrict__ row_scale) {
    extern __shared__ float ex_x[];                  // [K]
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* xr = x + (size_t)(r / top) * x_stride;
    const float xs = row_scale != nullptr ? row_scale[r] : 1.0f;
    for (int c = threadIdx.x; c < K; c += blockDim.x) ex_x[ex_place<T>(c, vec != 0)] = dl_to_f32<T>(xr[c]) * xs;
    __syncthreads();
    const int e = ids[r];
    const int n0 = blockIdx.y * per_block;
    const int n1 = min(ff, n0 + per_block);
    const bool ok = e >= 0 && e < E;
    const bool gated = dl_gate_is_gated(kind);
    if (!ok) {                                       // no such expert (or one without matrices): nothing to compute
        for (int n = n0 + threadIdx.x; n < n1; n += blockDim.x) out[(size_t)r * ff + n] = dl_from_f32<T>(0.f);
        return;
    }
    const T* we = w + (size_t)(ok ? e : 0) * (gated ? 2 : 1) * ff * K;
    for (int n = n0 + warp; n < n1; n += EX_WARPS) {
        const T* gr = we + (size_t)n * K;
        const T* ur = we + (size_t)((gated ? ff : 0) + n) * K;
        const float g = gated ? ex_row_dot<T>(gr, ex_x, K, lane, vec != 0) : 0.f;
        const float u = ex_row_dot<T>(ur, ex_x, K, lane, vec != 0);
        if (lane == 0) out[(size_t)r * ff + n] = dl_from_f32<T>(ok ? dl_gate_value(kind, g, u, limit, alpha) : 0.f);
    }
}

extern "C" int dl_expert_gate_up(const void* x, int x_stride, const int32_t* ids, const void* w, void* out, int dtype,
                                 int tokens, int top, int K, int ff, int E, int kind, float limit, float alpha,
                                 const float* row_scale, void* stream) {
    DL_REQUIRE(tokens >= 0 && top > 0 && K > 0 && ff > 0 && E > 0 && x_stride >= K && kind >= 0 && kind < GATE_KINDS,
               "expert_gate_up: bad arguments");
    DL_REQUIRE(ex_staged(K, 8) * sizeof(float) <= 48 * 1024, "expert_gate_up: rows of %d values are more than the kernel takes", K);
    if (tokens == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int per_block = ex_outputs_per_block(tokens * top, ff);
    const dim3 grid(tokens * top, (ff + per_block - 1) / per_block), block(32 * EX_WARPS);
    const size_t smem = ex_staged(K, 8) * sizeof(float);
    const int vec = (K % 8 == 0 && ((uintptr_t)w % 16) == 0) ? 1 : 0;      // every weight row starts on a 16-byte boundary
    cudaError_t e;
    if (dtype == DL_F32)
        e = dl_launch_dependent(expert_gate_up_kernel<float>, grid, block, smem, s, (const float*)x, x_stride, ids, (const float*)w,
                                (float*)out, top, K, ff, E, kind, limit, alpha, vec, per_block, row_scale);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(expert_gate_up_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)x, x_stride, ids,
                                (const __nv_bfloat16*)w, (__nv_bfloat16*)out, top, K, ff, E, kind, limit, alpha, vec, per_block, row_scale);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "expert_gate_up: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "expert_gate_up: %s", cudaGetErrorString(e));
    return DL_OK;
}

// out[t, n] = sum_j weights[t, j] * (D_e(t,j)[n, :] . h[t * top + j, :])  (+ addend[t, n]), float32.
// h: [tokens * top, ff] of dtype; w: [E, N, ff].  weights NULL: every weight is 1.  addend_gate (float32, one logit per
// token, addend_gate_stride apart) or NULL: the addend is multiplied by sigmoid(logit).  identity (rows identity_stride apart)
// or NULL: a chosen id in [E, E + n_identity) is an expert that gives back its input, weight * identity[t, n].
template <typename T>
__global__ void __launch_bounds__(32 * EX_WARPS)
expert_down_kernel(const T* __restrict__ h, const int32_t* __restrict__ ids, const float* __restrict__ weights,
                   const T* __restrict__ w, const float* __restrict__ addend, int addend_stride, float* __restrict__ out,
                   int top, int ff, int N, int E, int vec, int per_block, const float* __restrict__ addend_gate,
                   int addend_gate_stride, const T* __restrict__ identity, int identity_stride, int n_identity) {
    extern __shared__ float ex_h[];                  // [top][ff]
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* hr = h + (size_t)t * top * ff;
    const int staged = vec ? (ff + 32 * ExVec<T>::N - 1) / (32 * ExVec<T>::N) * 32 * ExVec<T>::N : ff;     // per choice
    for (int c = threadIdx.x; c < top * ff; c += blockDim.x) {
        const int j = c / ff;
        ex_h[(size_t)j * staged + ex_place<T>(c - j * ff, vec != 0)] = dl_to_f32<T>(hr[c]);
    }
    __syncthreads();
    const int n0 = blockIdx.y * per_block;
    const int n1 = min(N, n0 + per_block);
    const float ag = addend_gate != nullptr ? 1.0f / (1.0f + expf(-addend_gate[(size_t)t * addend_gate_stride])) : 1.0f;
    for (int n = n0 + warp; n < n1; n += EX_WARPS) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = ids[(size_t)t * top + j];
            if (e >= E && e < E + n_identity && identity != nullptr)
                total += (weights != nullptr ? weights[(size_t)t * top + j] : 1.0f) * dl_to_f32<T>(identity[(size_t)t * identity_stride + n]);
            if (e < 0 || e >= E) continue;
            const T* wr = w + ((size_t)e * N + n) * ff;
            const float* hj = ex_h + (size_t)j * staged;
            total += (weights != nullptr ? weights[(size_t)t * top + j] : 1.0f) * ex_row_dot<T>(wr, hj, ff, lane, vec != 0);
        }
        if (lane == 0) out[(size_t)t * N + n] = total + (addend != nullptr ? ag * addend[(size_t)t * addend_stride + n] : 0.f);
    }
}

extern "C" int dl_expert_down(const void* h, const int32_t* ids, const float* weights, const void* w, const float* addend,
                              int addend_stride, float* out, int dtype, int tokens, int top, int ff, int N, int E,
                              const float* addend_gate, int addend_gate_stride, const void* identity, int identity_stride,
                              int n_identity, void* stream) {
    DL_REQUIRE(tokens >= 0 && top > 0 && ff > 0 && N > 0 && E > 0, "expert_down: bad sizes");
    DL_REQUIRE(identity == nullptr || (n_identity > 0 && identity_stride >= N), "expert_down: identity experts give back rows of the output's width");
    DL_REQUIRE((size_t)top * ex_staged(ff, 8) * sizeof(float) <= 96 * 1024, "expert_down: %d x %d activations are more than the kernel takes",
               top, ff);
    if (tokens == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int per_block = ex_outputs_per_block(tokens, N);
    const dim3 grid(tokens, (N + per_block - 1) / per_block), block(32 * EX_WARPS);
    const size_t smem = (size_t)top * ex_staged(ff, 8) * sizeof(float);
    const int vec = (ff % 8 == 0 && ((uintptr_t)w % 16) == 0) ? 1 : 0;
    cudaError_t e;
    if (dtype == DL_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(expert_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = dl_launch_dependent(expert_down_kernel<float>, grid, block, smem, s, (const float*)h, ids, weights, (const float*)w,
                                addend, addend_stride, out, top, ff, N, E, vec, per_block, addend_gate, addend_gate_stride,
                                (const float*)identity, identity_stride, n_identity);
    } else if (dtype == DL_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(expert_down_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = dl_launch_dependent(expert_down_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)h, ids, weights,
                                (const __nv_bfloat16*)w, addend, addend_stride, out, top, ff, N, E, vec, per_block, addend_gate,
                                addend_gate_stride, (const __nv_bfloat16*)identity, identity_stride, n_identity);
    } else
        return dl_fail(DL_ERR_UNSUPPORTED, "expert_down: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "expert_down: %s", cudaGetErrorString(e));
    return DL_OK;
}

// ---------------------------------------------------------------------------------------------
// Many rows (a prompt, a large decode batch): the rows are sorted by expert so that a tensor-core
// product can take an expert's rows as tiles (dl_gemm_tc_grouped_bf16).  Everything is decided on the
// device: one block counts the rows of each expert, lays the experts' runs out one behind the other,
// each padded to whole tiles of EX_TILE rows, gives every (token, choice) row its place in its
// expert's run, and names each tile's expert.  Which place within a run a row gets depends on the
// order in which threads arrive; no result depends on it (a row's products do not depend on the
// other rows of its tile).
#define EX_TILE 128
#define EX_SORT_THREADS 1024

__global__ void __launch_bounds__(EX_SORT_THREADS)
expert_sort_kernel(const int32_t* __restrict__ ids, int rows, int E, int32_t* __restrict__ place, int32_t* __restrict__ tile_expert,
                   int max_tiles) {
    extern __shared__ int sort_smem[];               // [E] counts, then [E] cursors
    int* counts = sort_smem;
    int* cursor = sort_smem + E;
    dl_launch_dependents();
    dl_grid_dependency_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = tile * EX_TILE;
            const int n = (counts[e] + EX_TILE - 1) / EX_TILE;
            for (int b = 0; b < n && tile < max_tiles; ++b) tile_expert[tile++] = e;
        }
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        const int e = ids[i];
        place[i] = (e >= 0 && e < E) ? atomicAdd(&cursor[e], 1) : -1;
    }
}

// sorted[place[r], :] = x[r / top, :]   (16 bytes a thread)
__global__ void __launch_bounds__(256)
expert_gather_kernel(const uint4* __restrict__ x, int x_stride16, const int32_t* __restrict__ place, uint4* __restrict__ sorted,
                     int top, int k16) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int r = blockIdx.x;
    const int p = place[r];
    if (p < 0) return;
    const uint4* src = x + (size_t)(r / top) * x_stride16;
    uint4* dst = sorted + (size_t)p * k16;
    for (int c = threadIdx.x; c < k16; c += blockDim.x) dst[c] = src[c];
}

// sorted[place[r], :] = x[r / top, :] * row_scale[r], the product taken in float32 and rounded once
__global__ void __launch_bounds__(256)
expert_gather_scaled_kernel(const uint4* __restrict__ x, int x_stride16, const int32_t* __restrict__ place, uint4* __restrict__ sorted,
                            int top, int k16, const float* __restrict__ row_scale) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int r = blockIdx.x;
    const int p = place[r];
    if (p < 0) return;
    const float xs = row_scale[r];
    const uint4* src = x + (size_t)(r / top) * x_stride16;
    uint4* dst = sorted + (size_t)p * k16;
    for (int c = threadIdx.x; c < k16; c += blockDim.x) {
        uint4 raw = src[c];
        __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __floats2bfloat162_rn(__low2float(v[i]) * xs, __high2float(v[i]) * xs);
        dst[c] = raw;
    }
}

// out[t, n] = sum_j weights[t, j] * y[place[t * top + j], n]  (+ addend[t, n]), float32; weights NULL: all 1;
// addend_gate and identity (bfloat16 rows; ids name the chosen experts, E of them with matrices) as in the down kernel above
__global__ void __launch_bounds__(256)
expert_combine_kernel(const float* __restrict__ y, int y_stride, const int32_t* __restrict__ place, const float* __restrict__ weights,
                      const float* __restrict__ addend, int addend_stride, float* __restrict__ out, int top, int N,
                      const float* __restrict__ addend_gate, int addend_gate_stride, const int32_t* __restrict__ ids,
                      const __nv_bfloat16* __restrict__ identity, int identity_stride, int E, int n_identity) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t = blockIdx.x;
    const float ag = addend_gate != nullptr ? 1.0f / (1.0f + expf(-addend_gate[(size_t)t * addend_gate_stride])) : 1.0f;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = place[(size_t)t * top + j];
            if (p >= 0) total += (weights != nullptr ? weights[(size_t)t * top + j] : 1.0f) * y[(size_t)p * y_stride + n];
            else if (identity != nullptr) {
                const int e = ids[(size_t)t * top + j];
                if (e >= E && e < E + n_identity)
                    total += (weights != nullptr ? weights[(size_t)t * top + j] : 1.0f) * __bfloat162float(identity[(size_t)t * identity_stride + n]);
            }
        }
        out[(size_t)t * N + n] = total + (addend != nullptr ? ag * addend[(size_t)t * addend_stride + n] : 0.f);
    }
}

// ids int32 [rows] (rows = tokens * top); place int32 [rows]; tile_expert int32 [max_tiles], max_tiles >= rows / 128 + E.
extern "C" int dl_expert_sort(const int32_t* ids, int rows, int E, int32_t* place, int32_t* tile_expert, int max_tiles, void* stream) {
    DL_REQUIRE(rows >= 0 && E > 0 && max_tiles >= (rows + EX_TILE - 1) / EX_TILE + E - 1, "expert_sort: %d tiles do not hold %d rows of %d experts",
               max_tiles, rows, E);
    DL_REQUIRE((size_t)2 * E * sizeof(int) <= 48 * 1024, "expert_sort: too many experts");
    cudaError_t e = dl_launch_dependent(expert_sort_kernel, dim3(1), dim3(EX_SORT_THREADS), (size_t)2 * E * sizeof(int),
                                        (cudaStream_t)stream, ids, rows, E, place, tile_expert, max_tiles);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "expert_sort: %s", cudaGetErrorString(e));
    return DL_OK;
}

// x bfloat16 [tokens, K] (rows x_stride apart, 16-byte aligned, K a multiple of 8); sorted bfloat16 [padded rows, K].
// row_scale float32 [rows] or NULL: a row is multiplied by its scale on the way.
extern "C" int dl_expert_gather(const void* x, int x_stride, const int32_t* place, void* sorted, int rows, int top, int K,
                                const float* row_scale, void* stream) {
    DL_REQUIRE(rows >= 0 && top > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)sorted % 16) == 0,
               "expert_gather: rows of a multiple of 8 bfloat16 values, 16-byte aligned");
    if (rows == 0) return DL_OK;
    cudaError_t e = row_scale != nullptr
        ? dl_launch_dependent(expert_gather_scaled_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const uint4*)x,
                              x_stride / 8, place, (uint4*)sorted, top, K / 8, row_scale)
        : dl_launch_dependent(expert_gather_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const uint4*)x,
                              x_stride / 8, place, (uint4*)sorted, top, K / 8);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "expert_gather: %s", cudaGetErrorString(e));
    return DL_OK;
}

extern "C" int dl_expert_combine(const float* y, int y_stride, const int32_t* place, const float* weights, const float* addend,
                                 int addend_stride, float* out, int tokens, int top, int N, const float* addend_gate,
                                 int addend_gate_stride, const int32_t* ids, const void* identity, int identity_stride, int E,
                                 int n_identity, void* stream) {
    DL_REQUIRE(tokens >= 0 && top > 0 && N > 0 && y_stride >= N, "expert_combine: bad sizes");
    DL_REQUIRE(identity == nullptr || (ids != nullptr && n_identity > 0 && identity_stride >= N), "expert_combine: identity experts need the ids");
    if (tokens == 0) return DL_OK;
    cudaError_t e = dl_launch_dependent(expert_combine_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, y, y_stride, place,
                                        weights, addend, addend_stride, out, top, N, addend_gate, addend_gate_stride, ids,
                                        (const __nv_bfloat16*)identity, identity_stride, E, n_identity);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "expert_combine: %s", cudaGetErrorString(e));
    return DL_OK;
}
