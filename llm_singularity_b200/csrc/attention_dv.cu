// Softmax attention over the paged cache for mixers whose keys and values have sizes of their own
// (dk for queries and keys, dv for values) and whose mask may be cut into chunks:
//
//   query row i of request r sits at position p = kv_len - q_len + i and sees the keys at
//   positions [lo, p], lo = max(window > 0 ? p - window + 1 : 0, chunk > 0 ? (p / chunk) * chunk : 0)
//
// (chunks are counted from position 0 of the sequence, wherever a prompt was cut).  Query head h
// reads kv head h / (nh / nkv); scores (q . k) * scale; softmax by running maximum and sum; the
// weighted sum of values is divided by the sum at the end and, if a gate is given, multiplied by
// sigmoid(gate[t, h * dv + c]) on the way out.  Keys are [page][kv head][offset][dk], values
// [page][kv head][offset][dv].  Scores, weights and sums are 32-bit.
//
// Generic form (any sizes, 32-bit or bfloat16 storage): one warp owns a (row, head); lanes split
// the keys of a 32-key stretch for the scores and the value dims for the weighted sum.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kDvWarps = 4;
constexpr int kDvMaxDim = 256;

template <typename T>
__device__ __forceinline__ float dv_dot(const float* __restrict__ q, const T* __restrict__ k, int n, bool vec) {
    float s = 0.f;
    if (vec) {
        if constexpr (sizeof(T) == 4) {
            for (int d = 0; d < n; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(k + d);
                s += q[d] * kv.x + q[d + 1] * kv.y + q[d + 2] * kv.z + q[d + 3] * kv.w;
            }
        } else {
            for (int d = 0; d < n; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(p[j]);
                    s += q[d + 2 * j] * f.x + q[d + 2 * j + 1] * f.y;
                }
            }
        }
    } else {
        for (int d = 0; d < n; ++d) s += q[d] * lsb_to_float(k[d]);
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(kDvWarps * 32)
attention_dv_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                            const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                            const int* __restrict__ table_rows, const int* __restrict__ block_table, int table_stride,
                            const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                            int nh, int nkv, int dk, int dv, int page_size, int num_pages, float scale, int window,
                            int chunk, int vec) {
    __shared__ float q_sh[kDvWarps][kDvMaxDim];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z, h = blockIdx.y;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int i = blockIdx.x * kDvWarps + warp;             // row within the request
    if (i >= q_len) return;                                  // whole warp leaves together
    const int kv_len = kv_len_arr[r];
    const int p = kv_len - q_len + i;
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
    const int g = h / (nh / nkv);
    const int t = qs + i;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;

    const T* qr = q + ((size_t)t * nh + h) * dk;
    for (int d = lane; d < dk; d += 32) q_sh[warp][d] = lsb_to_float(qr[d]) * scale;
    __syncwarp();

    constexpr int kAccs = kDvMaxDim / 32;
    float acc[kAccs];
#pragma unroll
    for (int c = 0; c < kAccs; ++c) acc[c] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    for (int base = lo; base <= p; base += 32) {
        const int kj = base + lane;
        float s = -FLT_MAX;
        long long at = -1;                                   // (page, kv head, offset) as a row number
        if (kj <= p) {
            const int page = bt[kj / page_size];
            if (page < 0 || page >= num_pages) {
                lsb_set_status(LSB_BAD_PAGE);
            } else {
                at = ((long long)page * nkv + g) * page_size + (kj % page_size);
                s = dv_dot<T>(q_sh[warp], k_pages + at * dk, dk, vec != 0);
            }
        }
        const float m_new = fmaxf(m, lsb_warp_max(s));
        const float corr = expf(m - m_new);                  // m == -FLT_MAX first: exp(-huge) = 0
        const float pj = (at >= 0) ? expf(s - m_new) : 0.f;
        l = l * corr + lsb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < kAccs; ++c) acc[c] *= corr;
        const int n_valid = min(32, p - base + 1);
        for (int j = 0; j < n_valid; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const long long vat = __shfl_sync(0xffffffffu, at, j);
            if (vat < 0) continue;
            const T* v = v_pages + vat * dv;
#pragma unroll
            for (int c = 0; c < kAccs; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) acc[c] += w * lsb_to_float(v[d]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + ((size_t)t * nh + h) * dv;
    const T* gr = gate ? gate + (size_t)t * gate_stride + (size_t)h * dv : nullptr;
#pragma unroll
    for (int c = 0; c < kAccs; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) {
            float y = acc[c] * inv;
            if (gr) y *= 1.f / (1.f + expf(-lsb_to_float(gr[d])));
            o[d] = lsb_from_float<T>(y);
        }
    }
}

LSB_API int lsb_attention_dv_max_dim() { return kDvMaxDim; }

// q [tokens, nh * dk], out [tokens, nh * dv]; gate (or null) has rows `gate_stride` elements apart
// with the nh * dv gate values first.
LSB_API int lsb_attention_dv_generic(const void* q, const void* k_pages, const void* v_pages, const int* q_start,
                                     const int* kv_len, const int* table_rows, const int* block_table,
                                     int table_stride, const void* gate, long long gate_stride, void* out, int dtype,
                                     int n_requests, int max_q_len, int nh, int nkv, int dk, int dv, int page_size,
                                     int num_pages, float scale, int window, int chunk, cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (dk <= 0 || dk > kDvMaxDim || dv <= 0 || dv > kDvMaxDim || nkv <= 0 || nh % nkv || window < 0 || chunk < 0)
        return (int)cudaErrorInvalidValue;
    if (n_requests > 65535 || nh > 65535) return (int)cudaErrorInvalidValue;
    const int al = dtype == LSB_F32 ? 4 : 8;
    const int vec = (dk % al == 0 && (uintptr_t)k_pages % 16 == 0) ? 1 : 0;
    dim3 grid((max_q_len + kDvWarps - 1) / kDvWarps, nh, n_requests);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        attention_dv_generic_kernel<T>, grid, dim3(kDvWarps * 32), 0, stream, 1, (const T*)q, (const T*)k_pages,
        (const T*)v_pages, q_start, kv_len, table_rows, block_table, table_stride, (const T*)gate, gate_stride,
        (T*)out, nh, nkv, dk, dv, page_size, num_pages, scale, window, chunk, vec));
    return 0;
}
