// RMSNorm over the float32 residual stream, with the residual add fused in.
//
//   y = x * (1 / sqrt(mean(x^2) + eps)) * gain          (eps inside the root)
//
// Same statistics as the reference's rmsnorm_f32 / fused_add_rmsnorm_f16
// (native/kernels/rmsnorm_f32.cu:3-36, native/kernels/fused_add_rmsnorm.cu:9-72): the sum
// of squares, the root and the add are float32; only the normalised output may be
// bfloat16.  One block per row, a fixed block size, so a row's rounding does not depend
// on the rest of the batch.
//
// Rows of up to 8192 values whose width is a multiple of 4 take the register path: every
// thread loads its float4 pieces at once (a decode step has a handful of rows, so the
// kernel's time is one round of memory latency, not a loop of them), keeps them in
// registers across the reduction, and reads nothing twice.  Other widths take the looped path.
#include "common.cuh"

#define NORM_THREADS 256
#define NORM_MAX_VEC 8            // float4 pieces per thread on the register path

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TDelta, typename TOut, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
                   const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    const int n_vec = width / 4;
    float4 v[NORM_MAX_VEC];
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n_vec) v[i] = Vec4<float>::load(residual + base + 4 * c);
    }
    if (ADD) {
#pragma unroll
        for (int i = 0; i < NORM_MAX_VEC; ++i) {
            const int c = threadIdx.x + i * NORM_THREADS;
            if (c < n_vec) {
                const float4 d = Vec4<TDelta>::load(delta + base + 4 * c);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                Vec4<float>::store(residual + base + 4 * c, v[i]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < n_vec) {
            const float4 gn = Vec4<float>::load(gain + 4 * c);
            Vec4<TOut>::store(out + base + 4 * c, make_float4(v[i].x * scale * gn.x, v[i].y * scale * gn.y,
                                                              v[i].z * scale * gn.z, v[i].w * scale * gn.w));
        }
    }
}

template <typename TDelta, typename TOut, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
               const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += NORM_THREADS) {
        float v = residual[base + c];
        if (ADD) {
            v += dl_to_f32<TDelta>(delta[base + c]);
            residual[base + c] = v;
        }
        ss += v * v;
    }
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += NORM_THREADS)
        out[base + c] = dl_from_f32<TOut>(residual[base + c] * scale * gain[c]);
}

template <typename TDelta, typename TOut>
static int launch_norm(float* residual, const void* delta, const float* gain, void* out, int rows, int width,
                       float eps, cudaStream_t s) {
    const bool aligned = ((uintptr_t)residual % 16 == 0) && ((uintptr_t)gain % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         (!delta || (uintptr_t)delta % 16 == 0);
    const bool vec = aligned && width % 4 == 0 && width <= 4 * NORM_THREADS * NORM_MAX_VEC;
    const TDelta* d = (const TDelta*)delta;
    TOut* o = (TOut*)out;
    cudaError_t e;
    const dim3 grid(rows), block(NORM_THREADS);
    const TDelta* none = nullptr;
    if (vec) {
        if (delta) e = dl_launch_dependent(rmsnorm_vec_kernel<TDelta, TOut, true>, grid, block, 0, s, residual, d, gain, o, width, eps);
        else e = dl_launch_dependent(rmsnorm_vec_kernel<TDelta, TOut, false>, grid, block, 0, s, residual, none, gain, o, width, eps);
    } else {
        if (delta) e = dl_launch_dependent(rmsnorm_kernel<TDelta, TOut, true>, grid, block, 0, s, residual, d, gain, o, width, eps);
        else e = dl_launch_dependent(rmsnorm_kernel<TDelta, TOut, false>, grid, block, 0, s, residual, none, gain, o, width, eps);
    }
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "rmsnorm: %s", cudaGetErrorString(e));
    return DL_OK;
}

// residual: float32 [rows, width], updated in place to residual + delta when delta != NULL.
// delta: [rows, width] of delta_dtype or NULL.  out: [rows, width] of out_dtype.
extern "C" int dl_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const float* gain, void* out,
                              int out_dtype, int rows, int width, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    DL_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool df = (delta_dtype == DL_F32), of = (out_dtype == DL_F32);
    DL_REQUIRE(df || delta_dtype == DL_BF16, "rmsnorm: delta dtype %d", delta_dtype);
    DL_REQUIRE(of || out_dtype == DL_BF16, "rmsnorm: out dtype %d", out_dtype);
    if (df && of) return launch_norm<float, float>(residual, delta, gain, out, rows, width, eps, s);
    if (df && !of) return launch_norm<float, __nv_bfloat16>(residual, delta, gain, out, rows, width, eps, s);
    if (!df && of) return launch_norm<__nv_bfloat16, float>(residual, delta, gain, out, rows, width, eps, s);
    return launch_norm<__nv_bfloat16, __nv_bfloat16>(residual, delta, gain, out, rows, width, eps, s);
}

// A branch output that is normalised before it joins the stream (a layer with a norm behind each
// sublayer as well as before it), fused with the norm that follows:
//
//   residual += delta / sqrt(mean(delta^2) + delta_eps) * delta_gain  (+ extra)
//   out       = residual / sqrt(mean(residual^2) + eps) * gain          (when out is given)
//
// One block per row, float32 statistics, a fixed order of additions per row.  `extra` (float32, same
// shape as the stream, or NULL) is added as it is: the embedding output that a repeated group of
// layers takes in again before each pass.  Rows of up to 4 * NORM_THREADS values keep the sum in
// registers between the passes; wider rows go through the stream in memory.
#define BRANCH_MAX 4

template <typename TDelta, typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
branch_norm_add_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta, int delta_stride,
                       const float* __restrict__ delta_gain, float delta_eps, const float* __restrict__ extra,
                       const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    const TDelta* drow = delta + (size_t)blockIdx.x * delta_stride;
    const bool in_regs = width <= BRANCH_MAX * NORM_THREADS;
    float d[BRANCH_MAX];
    float ssd = 0.f;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < BRANCH_MAX; ++i) {
            const int c = threadIdx.x + i * NORM_THREADS;
            d[i] = c < width ? dl_to_f32<TDelta>(drow[c]) : 0.f;
            ssd += d[i] * d[i];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += NORM_THREADS) {
            const float v = dl_to_f32<TDelta>(drow[c]);
            ssd += v * v;
        }
    }
    ssd = dl_block_sum(ssd, scratch);
    const float dscale = 1.0f / sqrtf(ssd / (float)width + delta_eps);
    float ss = 0.f;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < BRANCH_MAX; ++i) {
            const int c = threadIdx.x + i * NORM_THREADS;
            if (c < width) {
                float v = residual[base + c] + d[i] * dscale * delta_gain[c];
                if (extra != nullptr) v += extra[base + c];
                residual[base + c] = v;
                d[i] = v;
                ss += v * v;
            }
        }
    } else {
        for (int c = threadIdx.x; c < width; c += NORM_THREADS) {
            float v = residual[base + c] + dl_to_f32<TDelta>(drow[c]) * dscale * delta_gain[c];
            if (extra != nullptr) v += extra[base + c];
            residual[base + c] = v;
            ss += v * v;
        }
    }
    if (out == nullptr) return;
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < BRANCH_MAX; ++i) {
            const int c = threadIdx.x + i * NORM_THREADS;
            if (c < width) out[base + c] = dl_from_f32<TOut>(d[i] * scale * gain[c]);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += NORM_THREADS)
            out[base + c] = dl_from_f32<TOut>(residual[base + c] * scale * gain[c]);
    }
}

template <typename TDelta, typename TOut>
static int launch_branch(float* residual, const void* delta, int delta_stride, const float* delta_gain, float delta_eps,
                         const float* extra, const float* gain, void* out, int rows, int width, float eps, cudaStream_t s) {
    cudaError_t e = dl_launch_dependent(branch_norm_add_kernel<TDelta, TOut>, dim3(rows), dim3(NORM_THREADS), 0, s, residual,
                                        (const TDelta*)delta, delta_stride, delta_gain, delta_eps, extra, gain, (TOut*)out,
                                        width, eps);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "branch_norm_add: %s", cudaGetErrorString(e));
    return DL_OK;
}

// residual float32 [rows, width] contiguous, updated in place; delta [rows, width] of delta_dtype, rows
// delta_stride elements apart; delta_gain, gain float32 [width]; extra float32 [rows, width] or NULL;
// out [rows, width] of out_dtype or NULL (then gain may be NULL too: the stream is only added to).
extern "C" int dl_branch_norm_add(float* residual, const void* delta, int delta_dtype, int delta_stride,
                                  const float* delta_gain, float delta_eps, const float* extra, const float* gain,
                                  void* out, int out_dtype, int rows, int width, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && delta_stride >= width, "branch_norm_add: bad sizes rows=%d width=%d", rows, width);
    DL_REQUIRE(delta_eps > 0.f && (out == nullptr || (eps > 0.f && gain != nullptr)), "branch_norm_add: eps must be positive");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool df = (delta_dtype == DL_F32), of = (out_dtype == DL_F32);
    DL_REQUIRE(df || delta_dtype == DL_BF16, "branch_norm_add: delta dtype %d", delta_dtype);
    DL_REQUIRE(of || out_dtype == DL_BF16, "branch_norm_add: out dtype %d", out_dtype);
    if (df && of) return launch_branch<float, float>(residual, delta, delta_stride, delta_gain, delta_eps, extra, gain, out, rows, width, eps, s);
    if (df && !of) return launch_branch<float, __nv_bfloat16>(residual, delta, delta_stride, delta_gain, delta_eps, extra, gain, out, rows, width, eps, s);
    if (!df && of) return launch_branch<__nv_bfloat16, float>(residual, delta, delta_stride, delta_gain, delta_eps, extra, gain, out, rows, width, eps, s);
    return launch_branch<__nv_bfloat16, __nv_bfloat16>(residual, delta, delta_stride, delta_gain, delta_eps, extra, gain, out, rows, width, eps, s);
}

// Stream += other, float32, elementwise (a stream that takes another in when no norm follows at once).
__global__ void __launch_bounds__(256) add_rows_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) a[i] += b[i];
}

extern "C" int dl_add_rows(float* a, const float* b, int rows, int width, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0, "add_rows: bad sizes");
    if (rows == 0) return DL_OK;
    const size_t n = (size_t)rows * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    cudaError_t e = dl_launch_dependent(add_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, a, b, n);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "add_rows: %s", cudaGetErrorString(e));
    return DL_OK;
}

// RMS norm of every head of a row on its own, with a gain shared by the heads: queries and keys before they meet.
//   y[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * gain[:]
// The row holds heads_a heads under gain_a and, behind them, heads_b heads under gain_b (a stacked projection's
// queries and keys), each `dim` wide.  One warp per (row, head); statistics and the product in float32.
template <typename T>
__global__ void __launch_bounds__(128)
head_rmsnorm_kernel(const T* __restrict__ x, int x_stride, T* __restrict__ y, int y_stride, const float* __restrict__ gain_a,
                    const float* __restrict__ gain_b, int rows, int heads_a, int heads_b, int dim, float eps) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int lane = threadIdx.x & 31, heads = heads_a + heads_b;
    const long idx = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= (long)rows * heads) return;
    const int t = (int)(idx / heads), h = (int)(idx % heads);
    const T* src = x + (size_t)t * x_stride + (size_t)h * dim;
    T* dst = y + (size_t)t * y_stride + (size_t)h * dim;
    const float* gain = h < heads_a ? gain_a : gain_b;
    float ss = 0.f;
    for (int j = lane; j < dim; j += 32) { const float v = dl_to_f32<T>(src[j]); ss += v * v; }
    ss = dl_warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int j = lane; j < dim; j += 32) dst[j] = dl_from_f32<T>(dl_to_f32<T>(src[j]) * scale * gain[j]);
}

// x, y [rows, (heads_a + heads_b) * dim] of `dtype`, rows x_stride / y_stride apart; gain_a, gain_b float32 [dim]
// (gain_b may be NULL when heads_b is 0).
extern "C" int dl_head_rmsnorm(const void* x, int x_stride, void* y, int y_stride, int dtype, const float* gain_a,
                               const float* gain_b, int rows, int heads_a, int heads_b, int dim, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && heads_a >= 0 && heads_b >= 0 && heads_a + heads_b > 0 && dim > 0 && eps > 0.f, "head_rmsnorm: bad sizes");
    DL_REQUIRE(gain_a != nullptr && (heads_b == 0 || gain_b != nullptr), "head_rmsnorm: a gain is missing");
    const int width = (heads_a + heads_b) * dim;
    DL_REQUIRE(x_stride >= width && y_stride >= width, "head_rmsnorm: rows overlap");
    if (rows == 0) return DL_OK;
    const long warps = (long)rows * (heads_a + heads_b);
    const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
    cudaError_t e;
    if (dtype == DL_F32)
        e = dl_launch_dependent(head_rmsnorm_kernel<float>, grid, block, 0, (cudaStream_t)stream, (const float*)x, x_stride,
                                (float*)y, y_stride, gain_a, gain_b, rows, heads_a, heads_b, dim, eps);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(head_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x,
                                x_stride, (__nv_bfloat16*)y, y_stride, gain_a, gain_b, rows, heads_a, heads_b, dim, eps);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "head_rmsnorm: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "head_rmsnorm: %s", cudaGetErrorString(e));
    return DL_OK;
}
