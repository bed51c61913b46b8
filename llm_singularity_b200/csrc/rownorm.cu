// Row-wise operations on the 32-bit residual stream for arrangements that norm after the sum,
// and the group norms of mixer outputs.  One thread block owns a row; sums of squares, roots,
// sigmoids and the products are 32-bit; a result is rounded only where it leaves as T.
//
//   post_group_norm   s = alpha * x + delta * sigmoid(gate + bias)      (gate optional)
//                     y = s / sqrt(mean_group(s^2) + eps) * w           (groups of the row)
//                     x <- y (or s, for arrangements that norm before the sublayer); copy <- T(y)
//   gather_group_norm out[i] = T(group norm of x[rows[i]])
//   unit_add          x += y / sqrt(mean(y^2) + eps) * w;  copy <- T(x)
//   rows_norm_gate    out = T(group norm of a 32-bit row, weight index modulo its length,
//                     times sigmoid(gate) if a gate is given)
//   cast_rows         out = T(x)
//   token_side_gate   out[t, j] = T(act(g[t, j]) * table[token[t], offset + j])
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kRowThreads = 256;

__device__ __forceinline__ float lsb_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }

// Sum of squares of each group of the row held in shared memory, every thread gets its group's
// factor through `factor` (shared, one float per group).
__device__ __forceinline__ void group_factors(const float* row, int n, int groups, float eps,
                                              float* factor, float* scratch) {
    const int gs = n / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const float v = row[g * gs + i];
            ss += v * v;
        }
        ss = lsb_block_sum(ss, scratch);
        if (threadIdx.x == 0) factor[g] = 1.f / sqrtf(ss / (float)gs + eps);
    }
    __syncthreads();
}

// four consecutive values as floats (16-byte or 8-byte accesses; the caller has checked alignment)
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
post_group_norm_kernel(float* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ gate,
                       long long gate_stride, const float* __restrict__ gate_bias,
                       const float* __restrict__ w, T* __restrict__ copy, int n, int groups,
                       float alpha, float eps, int keep_sum, int vec) {
    extern __shared__ float sh[];
    float* row = sh;                 // n
    float* factor = sh + n;          // groups
    float* scratch = factor + groups;
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    if (vec) {
        // four values a thread and pass (n is a multiple of four, group borders too)
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            float s[4], d[4], z[4], b[4];
            load4(x + t * n + i, s);
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] *= alpha;
            if (delta) {
                load4(delta + t * n + i, d);
                if (gate) {
                    load4(gate + t * gate_stride + i, z);
                    if (gate_bias) {
                        load4(gate_bias + i, b);
#pragma unroll
                        for (int k = 0; k < 4; ++k) z[k] += b[k];
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) d[k] *= lsb_sigmoid(z[k]);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) s[k] += d[k];
            }
            store4(row + i, s);
        }
        __syncthreads();
        group_factors(row, n, groups, eps, factor, scratch);
        const int gs4 = n / groups;
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            float s[4], w4[4], y[4];
            load4(row + i, s);
            load4(w + i, w4);
            const float f = factor[i / gs4];
#pragma unroll
            for (int k = 0; k < 4; ++k) y[k] = s[k] * f * w4[k];
            store4(x + t * n + i, keep_sum ? s : y);
            if (copy) store4(copy + t * n + i, y);
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float s = alpha * x[t * n + i];
        if (delta) {
            float d = lsb_to_float(delta[t * n + i]);
            if (gate) {
                float z = lsb_to_float(gate[t * gate_stride + i]);
                if (gate_bias) z += gate_bias[i];
                d *= lsb_sigmoid(z);
            }
            s += d;
        }
        row[i] = s;
    }
    __syncthreads();
    group_factors(row, n, groups, eps, factor, scratch);
    const int gs = n / groups;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float y = row[i] * factor[i / gs] * w[i];
        x[t * n + i] = keep_sum ? row[i] : y;
        if (copy) copy[t * n + i] = lsb_from_float<T>(y);
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
gather_group_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, int n_rows_x,
                         const float* __restrict__ w, T* __restrict__ out, int n, int groups, float eps) {
    extern __shared__ float sh[];
    float* row = sh;
    float* factor = sh + n;
    float* scratch = factor + groups;
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = rows[blockIdx.x];
    if (r < 0 || r >= n_rows_x) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = x[(size_t)r * n + i];
    __syncthreads();
    group_factors(row, n, groups, eps, factor, scratch);
    const int gs = n / groups;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        out[(size_t)blockIdx.x * n + i] = lsb_from_float<T>(row[i] * factor[i / gs] * w[i]);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
unit_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ w,
                T* __restrict__ copy, int n, float eps) {
    extern __shared__ float sh[];
    float* row = sh;
    float* scratch = sh + n;
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = lsb_to_float(y[t * n + i]);
        row[i] = v;
        ss += v * v;
    }
    ss = lsb_block_sum(ss, scratch);
    const float f = 1.f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[t * n + i] + row[i] * f * w[i];
        x[t * n + i] = v;
        if (copy) copy[t * n + i] = lsb_from_float<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
rows_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_len,
                      const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                      int n, int groups, float eps) {
    extern __shared__ float sh[];
    float* row = sh;
    float* factor = sh + n;
    float* scratch = factor + groups;
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = x[t * n + i];
    __syncthreads();
    group_factors(row, n, groups, eps, factor, scratch);
    const int gs = n / groups;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = row[i] * factor[i / gs] * w[i % w_len];
        if (gate) y *= lsb_sigmoid(lsb_to_float(gate[t * gate_stride + i]));
        out[t * n + i] = lsb_from_float<T>(y);
    }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long count) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = lsb_from_float<T>(x[i]);
}

__device__ __forceinline__ float side_act(float z, int act) {
    if (act == 1) return z / (1.f + expf(-z));                                       // silu
    if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z;
}

template <typename T>
__global__ void token_side_gate_kernel(const T* __restrict__ g, const T* __restrict__ table,
                                       const int* __restrict__ tokens, T* __restrict__ out,
                                       int n_tokens, int dim, int table_cols, int offset, int vocab,
                                       int act) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const long long count = (long long)n_tokens * dim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / dim), j = (int)(i % dim);
        const int tok = tokens[t];
        if (tok < 0 || tok >= vocab) {
            lsb_set_status(LSB_BAD_TOKEN);
            out[i] = lsb_from_float<T>(0.f);
            continue;
        }
        const float e = lsb_to_float(table[(size_t)tok * table_cols + offset + j]);
        out[i] = lsb_from_float<T>(side_act(lsb_to_float(g[i]), act) * e);
    }
}

static inline size_t row_smem(int n, int groups) { return (size_t)(n + groups + 33) * sizeof(float); }

template <typename K>
static inline int allow_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

LSB_API int lsb_post_group_norm(float* x, const void* delta, const void* gate, long long gate_stride,
                                const float* gate_bias, const float* w, void* copy, int dtype,
                                int rows, int n, int groups, float alpha, float eps, int keep_sum,
                                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || groups <= 0 || n % groups || row_smem(n, groups) > 200 * 1024) return (int)cudaErrorInvalidValue;
    const size_t smem = row_smem(n, groups);
    LSB_DISPATCH_DTYPE(dtype, {
        int rc = allow_smem(post_group_norm_kernel<T>, smem);
        if (rc) return rc;
        // vector accesses: groups of four values that never straddle a norm group, all rows aligned
        const size_t esz = sizeof(T);
        const int vec = (n % 4 == 0 && (n / groups) % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                         (uintptr_t)delta % (4 * esz) == 0 && (uintptr_t)copy % (4 * esz) == 0 &&
                         (uintptr_t)gate % (4 * esz) == 0 && gate_stride % 4 == 0 && (uintptr_t)gate_bias % 16 == 0) ? 1 : 0;
        return lsb_launch(post_group_norm_kernel<T>, dim3(rows), dim3(kRowThreads), smem, stream, 1,
                          x, (const T*)delta, (const T*)gate, gate_stride, gate_bias, w, (T*)copy, n,
                          groups, alpha, eps, keep_sum, vec);
    });
    return 0;
}

LSB_API int lsb_gather_group_norm(const float* x, const int* rows, int n_rows, int n_rows_x,
                                  const float* w, void* out, int dtype, int n, int groups, float eps,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n <= 0 || groups <= 0 || n % groups || row_smem(n, groups) > 200 * 1024) return (int)cudaErrorInvalidValue;
    const size_t smem = row_smem(n, groups);
    LSB_DISPATCH_DTYPE(dtype, {
        int rc = allow_smem(gather_group_norm_kernel<T>, smem);
        if (rc) return rc;
        return lsb_launch(gather_group_norm_kernel<T>, dim3(n_rows), dim3(kRowThreads), smem, stream, 1,
                          x, rows, n_rows_x, w, (T*)out, n, groups, eps);
    });
    return 0;
}

LSB_API int lsb_unit_add(float* x, const void* y, const float* w, void* copy, int dtype, int rows, int n,
                         float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || row_smem(n, 0) > 200 * 1024) return (int)cudaErrorInvalidValue;
    const size_t smem = row_smem(n, 0);
    LSB_DISPATCH_DTYPE(dtype, {
        int rc = allow_smem(unit_add_kernel<T>, smem);
        if (rc) return rc;
        return lsb_launch(unit_add_kernel<T>, dim3(rows), dim3(kRowThreads), smem, stream, 1,
                          x, (const T*)y, w, (T*)copy, n, eps);
    });
    return 0;
}

LSB_API int lsb_rows_norm_gate(const float* x, const float* w, int w_len, const void* gate,
                               long long gate_stride, void* out, int dtype, int rows, int n, int groups,
                               float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || groups <= 0 || n % groups || w_len <= 0 || row_smem(n, groups) > 200 * 1024)
        return (int)cudaErrorInvalidValue;
    const size_t smem = row_smem(n, groups);
    LSB_DISPATCH_DTYPE(dtype, {
        int rc = allow_smem(rows_norm_gate_kernel<T>, smem);
        if (rc) return rc;
        return lsb_launch(rows_norm_gate_kernel<T>, dim3(rows), dim3(kRowThreads), smem, stream, 1,
                          x, w, w_len, (const T*)gate, gate_stride, (T*)out, n, groups, eps);
    });
    return 0;
}

LSB_API int lsb_cast_rows(const float* x, void* out, int dtype, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    const int blocks = (int)((count + 1023) / 1024 < 2048 ? (count + 1023) / 1024 : 2048);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(cast_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, 1,
                                                x, (T*)out, count));
    return 0;
}

LSB_API int lsb_token_side_gate(const void* g, const void* table, const int* tokens, void* out, int dtype,
                                int n_tokens, int dim, int table_cols, int offset, int vocab, int act,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || offset < 0 || offset + dim > table_cols) return (int)cudaErrorInvalidValue;
    const long long count = (long long)n_tokens * dim;
    const int blocks = (int)((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(token_side_gate_kernel<T>, dim3(blocks), dim3(256), 0, stream, 1,
                                                (const T*)g, (const T*)table, tokens, (T*)out, n_tokens,
                                                dim, table_cols, offset, vocab, act));
    return 0;
}
