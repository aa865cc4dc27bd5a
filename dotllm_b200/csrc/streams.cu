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
#define ST_MAX_COPIES 16

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

// The same pass for rows of up to 4 * ST_THREADS * ST_MAX_VEC values whose width is a multiple of 4, and up to four copies:
// every thread loads its 16-byte pieces of all copies and of y at once (a decode step has a handful of rows, so the
// kernel's time is one round of memory latency, not a loop of them) and keeps its pieces of u in registers across the two
// reductions.  The arithmetic per value and its order are the looped kernel's; the block sums add the same partial sums in
// another order.
#define ST_MAX_VEC 8

template <typename T> struct StVec4;
template <> struct StVec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct StVec4<__nv_bfloat16> {
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

__device__ __forceinline__ float4 st_fma4(float a, float4 x, float4 acc) {
    return make_float4(fmaf(a, x.x, acc.x), fmaf(a, x.y, acc.y), fmaf(a, x.z, acc.z), fmaf(a, x.w, acc.w));
}

template <typename TY, typename TOut, int S, int NV>
__global__ void __launch_bounds__(ST_THREADS)
stream_norm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, int y_stride, const float* __restrict__ scale,
                       const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ read,
                       const float* __restrict__ gain, const float* __restrict__ bias, TOut* __restrict__ normed,
                       float* __restrict__ summed, int width, float eps, int kind) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    float w_mix[S * S], w_out[S], w_read[S];
#pragma unroll
    for (int i = 0; i < S * S; ++i) w_mix[i] = mix != nullptr ? mix[i] : 0.f;
#pragma unroll
    for (int i = 0; i < S; ++i) { w_out[i] = outw != nullptr ? outw[i] : 0.f; w_read[i] = read != nullptr ? read[i] : 1.f; }
    dl_grid_dependency_wait();
    float* row = x + (size_t)blockIdx.x * S * width;
    const int n_vec = width / 4;
    const bool write = y != nullptr;
    float4 u[NV];
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * ST_THREADS;
        u[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c >= n_vec) continue;
        float4 old[S];
#pragma unroll
        for (int s = 0; s < S; ++s) old[s] = StVec4<float>::load(row + (size_t)s * width + 4 * c);
        if (write) {
            float4 yy = StVec4<TY>::load(y + (size_t)blockIdx.x * y_stride + 4 * c);
            if (scale != nullptr) {
                const float4 sc = StVec4<float>::load(scale + 4 * c);
                yy = make_float4(yy.x * sc.x, yy.y * sc.y, yy.z * sc.z, yy.w * sc.w);
            }
#pragma unroll
            for (int t = 0; t < S; ++t) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < S; ++s) acc = st_fma4(w_mix[s * S + t], old[s], acc);
                acc = st_fma4(w_out[t], yy, acc);
                StVec4<float>::store(row + (size_t)t * width + 4 * c, acc);
                u[i] = st_fma4(w_read[t], acc, u[i]);
            }
        } else {
#pragma unroll
            for (int t = 0; t < S; ++t) u[i] = st_fma4(w_read[t], old[t], u[i]);
        }
        if (summed != nullptr) StVec4<float>::store(summed + (size_t)blockIdx.x * width + 4 * c, u[i]);
        total += kind == 0 ? (u[i].x + u[i].y) + (u[i].z + u[i].w) : (u[i].x * u[i].x + u[i].y * u[i].y) + (u[i].z * u[i].z + u[i].w * u[i].w);
    }
    if (normed == nullptr) return;
    total = dl_block_sum(total, scratch);
    float mean = 0.f, factor;
    if (kind == 0) {
        mean = total / (float)width;
        float dev = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (threadIdx.x + i * ST_THREADS >= n_vec) continue;
            const float a = u[i].x - mean, b = u[i].y - mean, c2 = u[i].z - mean, d = u[i].w - mean;
            dev += (a * a + b * b) + (c2 * c2 + d * d);
        }
        dev = dl_block_sum(dev, scratch);
        factor = 1.0f / sqrtf(dev / (float)width + eps);
    } else {
        factor = 1.0f / sqrtf(total / (float)width + eps);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * ST_THREADS;
        if (c >= n_vec) continue;
        const float4 gn = StVec4<float>::load(gain + 4 * c);
        const float4 bs = bias != nullptr ? StVec4<float>::load(bias + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        StVec4<TOut>::store(normed + (size_t)blockIdx.x * width + 4 * c,
                            make_float4((u[i].x - mean) * factor * gn.x + bs.x, (u[i].y - mean) * factor * gn.y + bs.y,
                                        (u[i].z - mean) * factor * gn.z + bs.z, (u[i].w - mean) * factor * gn.w + bs.w));
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
    DL_REQUIRE(normed == nullptr || out_dtype == DL_F32 || out_dtype == DL_BF16, "stream_norm: out dtype %d", out_dtype);
    const auto aligned = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
    const bool vec = S <= 4 && width % 4 == 0 && width <= 4 * ST_THREADS * ST_MAX_VEC && aligned(x) && aligned(scale) && aligned(gain) &&
                     aligned(bias) && aligned(normed) && aligned(summed) && (y == nullptr || (aligned(y) && y_stride % 4 == 0));
    if (vec) {
        const int nv = (width / 4 + ST_THREADS - 1) / ST_THREADS;           // 16-byte pieces a thread
#define ST_VEC3(TY, TOUT, SS, NV)                                                                                            \
        e = dl_launch_dependent(stream_norm_vec_kernel<TY, TOUT, SS, NV>, grid, block, 0, s, x, (const TY*)y, y_stride, scale, mix,   \
                                outw, read, gain, bias, (TOUT*)normed, summed, width, eps, kind)
#define ST_VEC2(TY, TOUT, SS)                                                                                                \
        do {                                                                                                                 \
            if (nv <= 1) ST_VEC3(TY, TOUT, SS, 1); else if (nv <= 2) ST_VEC3(TY, TOUT, SS, 2);                               \
            else if (nv <= 4) ST_VEC3(TY, TOUT, SS, 4); else ST_VEC3(TY, TOUT, SS, ST_MAX_VEC);                             \
        } while (0)
#define ST_VEC1(TY, TOUT)                                                                                                    \
        do {                                                                                                                 \
            if (S == 1) ST_VEC2(TY, TOUT, 1); else if (S == 2) ST_VEC2(TY, TOUT, 2);                                         \
            else if (S == 3) ST_VEC2(TY, TOUT, 3); else ST_VEC2(TY, TOUT, 4);                                                \
        } while (0)
        const bool out16 = normed != nullptr && out_dtype == DL_BF16;
        if (y16 && out16) ST_VEC1(__nv_bfloat16, __nv_bfloat16);
        else if (y16) ST_VEC1(__nv_bfloat16, float);
        else if (out16) ST_VEC1(float, __nv_bfloat16);
        else ST_VEC1(float, float);
#undef ST_VEC1
#undef ST_VEC2
#undef ST_VEC3
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "stream_norm: %s", cudaGetErrorString(e));
        return DL_OK;
    }
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

// dst[r, s, :] = table[ids[r], :] * factor for every copy s, float32: the embedding straight into a stream of S copies.  An id
// outside the table gives a row of zeros.
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
embed_copies_kernel(const T* __restrict__ table, int table_stride, const int32_t* __restrict__ ids, float* __restrict__ dst, int S,
                    int width, int n_table_rows, float factor) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int id = ids[blockIdx.x];
    const bool ok = id >= 0 && id < n_table_rows;
    const T* src = table + (size_t)(ok ? id : 0) * table_stride;
    for (int c = threadIdx.x; c < width; c += ST_THREADS) {
        const float v = ok ? dl_to_f32<T>(src[c]) * factor : 0.f;
        for (int s = 0; s < S; ++s) dst[((size_t)blockIdx.x * S + s) * width + c] = v;
    }
}

extern "C" int dl_embed_copies(const void* table, int dtype, int table_stride, const int32_t* ids, float* dst, int rows, int S,
                               int width, int n_table_rows, float factor, void* stream) {
    DL_REQUIRE(rows >= 0 && S > 0 && width > 0 && n_table_rows > 0 && table_stride >= width, "embed_copies: bad sizes");
    if (rows == 0) return DL_OK;
    cudaError_t e;
    if (dtype == DL_F32)
        e = dl_launch_dependent(embed_copies_kernel<float>, dim3(rows), dim3(ST_THREADS), 0, (cudaStream_t)stream, (const float*)table,
                                table_stride, ids, dst, S, width, n_table_rows, factor);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(embed_copies_kernel<__nv_bfloat16>, dim3(rows), dim3(ST_THREADS), 0, (cudaStream_t)stream,
                                (const __nv_bfloat16*)table, table_stride, ids, dst, S, width, n_table_rows, factor);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "embed_copies: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "embed_copies: %s", cudaGetErrorString(e));
    return DL_OK;
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
