// A residual stream kept as several copies (hyper-connections), and the norms around it.
//
// The stream of a token is S copies x_1 .. x_S of `width` float32 values, side by side in one row [S * width].  A
// sublayer reads a weighted sum of the copies and writes its output back into all of them:
//
//   u      = sum_s read[s] x_s                     what the sublayer's norm sees
//   x_t   <- sum_s mix[s, t] x_s + out[t] * (scale .* y)     every copy at once, from the old copies
//
// with `scale` a gain per channel on the sublayer's output y (a layer scale; NULL for none).  S = 1 with mix = [[1]],
// out = [1] and read = [1] is the ordinary residual sum.  dl_stream_norm does, for one row per block: the write of the
// sublayer that ran last (when there is one), then the read for the sublayer that runs next and its norm -
//
//   kind 0 (layer norm):  (u - mean) / sqrt(mean((u - mean)^2) + eps) * gain + bias
//   kind 1 (RMS norm):     u / sqrt(mean(u^2) + eps) * gain
//
// - so the stream is read and written once per sublayer.  Everything is float32 except the normalised output (and y,
// which may come in bfloat16); the mean of the squared deviations is taken from the deviations themselves, which
// wait in shared memory.  A row's arithmetic and its order depend on the sizes alone.
//
// Also here: the RMS norm over groups of columns of a projection (queries and keys normalised over all their heads
// at once), the mean of two branches that are each RMS-normalised over the row, and a plain multiplication.
#include "common.cuh"

#define ST_THREADS 256
#define ST_MAX_COPIES 8

template <typename TY, typename TOut>
__global__ void __launch_bounds__(ST_THREADS)
stream_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, int y_stride, const float* __restrict__ scale,
                   const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ read,
                   const float* __restrict__ gain, const float* __restrict__ bias, TOut* __restrict__ normed,
                   float* __restrict__ summed, int S, int width, float eps, int kind) {
    extern __shared__ float st_u[];                    // [width]: the row the norm sees
    __shared__ float scratch[33];
    __shared__ float s_mix[ST_MAX_COPIES * ST_MAX_COPIES], s_out[ST_MAX_COPIES], s_read[ST_MAX_COPIES];
    dl_launch_dependents();
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix != nullptr ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = outw != nullptr ? outw[threadIdx.x] : 0.f;
        s_read[threadIdx.x] = read != nullptr ? read[threadIdx.x] : 1.f;
    }
    dl_grid_dependency_wait();
    __syncthreads();
    float* row = x + (size_t)blockIdx.x * S * width;
    const bool write = y != nullptr;
    float total = 0.f;
    for (int c = threadIdx.x; c < width; c += ST_THREADS) {
        float old[ST_MAX_COPIES];
#pragma unroll
        for (int s = 0; s < ST_MAX_COPIES; ++s) old[s] = s < S ? row[(size_t)s * width + c] : 0.f;
        float u = 0.f;
        if (write) {
            const float yy = dl_to_f32<TY>(y[(size_t)blockIdx.x * y_stride + c]) * (scale != nullptr ? scale[c] : 1.f);
#pragma unroll
            for (int t = 0; t < ST_MAX_COPIES; ++t) {
                if (t >= S) break;
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < ST_MAX_COPIES; ++s)
                    if (s < S) acc = fmaf(s_mix[s * S + t], old[s], acc);
                acc = fmaf(s_out[t], yy, acc);
                row[(size_t)t * width + c] = acc;
                u = fmaf(s_read[t], acc, u);
            }
        } else {
#pragma unroll
            for (int t = 0; t < ST_MAX_COPIES; ++t)
                if (t < S) u = fmaf(s_read[t], old[t], u);
        }
        st_u[c] = u;
        total += kind == 0 ? u : u * u;
    }
    if (summed != nullptr)
        for (int c = threadIdx.x; c < width; c += ST_THREADS) summed[(size_t)blockIdx.x * width + c] = st_u[c];
    if (normed == nullptr) return;
    total = dl_block_sum(total, scratch);
    float mean = 0.f, factor;
    if (kind == 0) {
        mean = total / (float)width;
        float dev = 0.f;
        for (int c = threadIdx.x; c < width; c += ST_THREADS) {
            const float d = st_u[c] - mean;
            dev += d * d;
        }
        dev = dl_block_sum(dev, scratch);
        factor = 1.0f / sqrtf(dev / (float)width + eps);
    } else {
        factor = 1.0f / sqrtf(total / (float)width + eps);
    }
    for (int c = threadIdx.x; c < width; c += ST_THREADS) {
        const float v = (st_u[c] - mean) * factor * gain[c] + (bias != nullptr ? bias[c] : 0.f);
        normed[(size_t)blockIdx.x * width + c] = dl_from_f32<TOut>(v);
    }
}

// x float32 [rows, S * width], updated in place when y is given; y [rows, width] of y_dtype (rows y_stride apart) or NULL
// (nothing is written); scale float32 [width] or NULL; mix float32 [S, S] (from, to), outw float32 [S] (both needed with
// y); read float32 [S] or NULL (every copy counts once); gain float32 [width], bias float32 [width] or NULL; normed
// [rows, width] of out_dtype or NULL (no norm); summed float32 [rows, width] or NULL (the read before the norm).
extern "C" int dl_stream_norm(float* x, const void* y, int y_dtype, int y_stride, const float* scale, const float* mix,
                              const float* outw, const float* read, const float* gain, const float* bias, void* normed,
                              int out_dtype, float* summed, int rows, int S, int width, float eps, int kind, void* stream) {
    DL_REQUIRE(rows >= 0 && S > 0 && S <= ST_MAX_COPIES && width > 0, "stream_norm: %d copies of %d values (up to %d copies)", S, width,
               ST_MAX_COPIES);
    DL_REQUIRE(kind == 0 || kind == 1, "stream_norm: norm kind %d (0: layer norm, 1: RMS norm)", kind);
    DL_REQUIRE(y == nullptr || (mix != nullptr && outw != nullptr && y_stride >= width), "stream_norm: a write needs mix and out weights");
    DL_REQUIRE(normed == nullptr || (gain != nullptr && eps > 0.f), "stream_norm: a norm needs a gain and a positive eps");
    DL_REQUIRE(normed != nullptr || summed != nullptr || y != nullptr, "stream_norm: nothing to do");
    const size_t smem = (size_t)width * sizeof(float);
    DL_REQUIRE(smem <= 160 * 1024, "stream_norm: rows of %d values are more than the kernel takes", width);
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(rows), block(ST_THREADS);
    cudaError_t e;
#define ST_LAUNCH(TY, TOUT)                                                                                                 \
    do {                                                                                                                    \
        if (smem > 48 * 1024)                                                                                               \
            cudaFuncSetAttribute(stream_norm_kernel<TY, TOUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        e = dl_launch_dependent(stream_norm_kernel<TY, TOUT>, grid, block, smem, s, x, (const TY*)y, y_stride, scale, mix,  \
                                outw, read, gain, bias, (TOUT*)normed, summed, S, width, eps, kind);                        \
    } while (0)
    const bool y16 = y != nullptr && y_dtype == DL_BF16;
    DL_REQUIRE(y == nullptr || y_dtype == DL_F32 || y_dtype == DL_BF16, "stream_norm: y dtype %d", y_dtype);
    if (normed == nullptr || out_dtype == DL_F32) {
        if (y16) ST_LAUNCH(__nv_bfloat16, float); else ST_LAUNCH(float, float);
    } else if (out_dtype == DL_BF16) {
        if (y16) ST_LAUNCH(__nv_bfloat16, __nv_bfloat16); else ST_LAUNCH(float, __nv_bfloat16);
    } else {
        return dl_fail(DL_ERR_UNSUPPORTED, "stream_norm: out dtype %d", out_dtype);
    }
#undef ST_LAUNCH
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "stream_norm: %s", cudaGetErrorString(e));
    return DL_OK;
}

// dst[r, s, :] = src[r, :] * factor for every copy s: the start of a stream of S copies.  src float32 [rows, width] -> dst
// [rows, S * width].
__global__ void __launch_bounds__(ST_THREADS)
stream_copies_kernel(const float* __restrict__ src, float* __restrict__ dst, int S, int width, float factor) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    for (int c = threadIdx.x; c < width; c += ST_THREADS) {
        const float v = src[(size_t)blockIdx.x * width + c] * factor;
        for (int s = 0; s < S; ++s) dst[((size_t)blockIdx.x * S + s) * width + c] = v;
    }
}

extern "C" int dl_stream_copies(const float* src, float* dst, int rows, int S, int width, float factor, void* stream) {
    DL_REQUIRE(rows >= 0 && S > 0 && width > 0, "stream_copies: bad sizes");
    if (rows == 0) return DL_OK;
    cudaError_t e = dl_launch_dependent(stream_copies_kernel, dim3(rows), dim3(ST_THREADS), 0, (cudaStream_t)stream, src, dst, S, width, factor);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "stream_copies: %s", cudaGetErrorString(e));
    return DL_OK;
}

// y[r, group g] = x[r, group g] / sqrt(mean over the group's columns of x^2 + eps) * gain[column]: a block per (row, group);
// group 0 is columns [0, width_a), group 1 columns [width_a, width_a + width_b).  gain float32 [width_a + width_b].
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
group_rmsnorm_kernel(const T* __restrict__ x, int x_stride, T* __restrict__ y, int y_stride, const float* __restrict__ gain,
                     int width_a, int width_b, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int first = blockIdx.y == 0 ? 0 : width_a, n = blockIdx.y == 0 ? width_a : width_b;
    const T* src = x + (size_t)blockIdx.x * x_stride + first;
    T* dst = y + (size_t)blockIdx.x * y_stride + first;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += ST_THREADS) { const float v = dl_to_f32<T>(src[c]); ss += v * v; }
    ss = dl_block_sum(ss, scratch);
    const float factor = 1.0f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += ST_THREADS) dst[c] = dl_from_f32<T>(dl_to_f32<T>(src[c]) * factor * gain[first + c]);
}

extern "C" int dl_group_rmsnorm(const void* x, int x_stride, void* y, int y_stride, int dtype, const float* gain, int rows,
                                int width_a, int width_b, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && width_a > 0 && width_b >= 0 && eps > 0.f && gain != nullptr, "group_rmsnorm: bad arguments");
    DL_REQUIRE(x_stride >= width_a + width_b && y_stride >= width_a + width_b, "group_rmsnorm: rows overlap");
    if (rows == 0) return DL_OK;
    const dim3 grid(rows, width_b > 0 ? 2 : 1), block(ST_THREADS);
    cudaError_t e;
    if (dtype == DL_F32)
        e = dl_launch_dependent(group_rmsnorm_kernel<float>, grid, block, 0, (cudaStream_t)stream, (const float*)x, x_stride, (float*)y,
                                y_stride, gain, width_a, width_b, eps);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(group_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x,
                                x_stride, (__nv_bfloat16*)y, y_stride, gain, width_a, width_b, eps);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "group_rmsnorm: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "group_rmsnorm: %s", cudaGetErrorString(e));
    return DL_OK;
}

// out[r, :] = wa * rms(a[r, :]) .* gain_a + wb * rms(b[r, :]) .* gain_b, float32; rms(v) = v / sqrt(mean(v^2) + eps).
__global__ void __launch_bounds__(ST_THREADS)
pair_norm_sum_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ gain_a,
                     const float* __restrict__ gain_b, float* __restrict__ out, int width, float eps, float wa, float wb) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const float* ra = a + (size_t)blockIdx.x * width;
    const float* rb = b + (size_t)blockIdx.x * width;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < width; c += ST_THREADS) { sa += ra[c] * ra[c]; sb += rb[c] * rb[c]; }
    sa = dl_block_sum(sa, scratch);
    sb = dl_block_sum(sb, scratch);
    const float fa = wa / sqrtf(sa / (float)width + eps), fb = wb / sqrtf(sb / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += ST_THREADS)
        out[(size_t)blockIdx.x * width + c] = ra[c] * fa * gain_a[c] + rb[c] * fb * gain_b[c];
}

extern "C" int dl_pair_norm_sum(const float* a, const float* b, const float* gain_a, const float* gain_b, float* out, int rows,
                                int width, float eps, float wa, float wb, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && eps > 0.f, "pair_norm_sum: bad arguments");
    if (rows == 0) return DL_OK;
    cudaError_t e = dl_launch_dependent(pair_norm_sum_kernel, dim3(rows), dim3(ST_THREADS), 0, (cudaStream_t)stream, a, b, gain_a,
                                        gain_b, out, width, eps, wa, wb);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "pair_norm_sum: %s", cudaGetErrorString(e));
    return DL_OK;
}

// values[i] *= factor, float32, in place
__global__ void __launch_bounds__(256) scale_values_kernel(float* __restrict__ values, long long n, float factor) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) values[i] *= factor;
}

extern "C" int dl_scale_values(float* values, long long n, float factor, void* stream) {
    DL_REQUIRE(n >= 0, "scale_values: bad size");
    if (n == 0) return DL_OK;
    cudaError_t e = dl_launch_dependent(scale_values_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                                        values, n, factor);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "scale_values: %s", cudaGetErrorString(e));
    return DL_OK;
}
