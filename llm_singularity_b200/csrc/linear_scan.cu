// The recurrence of linear attention with a matrix state per head:
//
//     S_t = diag(a_t) S_(t-1) + b_t v_t^T          o_t = S_t^T q_t
//
// for any mix of prompt portions and single decode tokens, each request continuing from the
// state its slot holds.  S is [key_dim, value_dim] per head, 32-bit, stored [slot, head,
// value_dim, key_dim] (key_dim contiguous).  Everything that enters the recurrence is formed in
// 32-bit here from the projections' outputs:
//
//   gate 0 (fixed decay):  a = decay[head] for every channel,  b = act_k(k projection)
//   gate 1 (forget gate):  a = floor + (1 - floor) * sigmoid(f projection + bias),  b = 1 - a
//   q = act_q(q projection), v = act_v(v projection); act: 0 none, 1 silu
//
// A block owns (request, head, a tile of value columns) and walks the request's tokens in order,
// so the result does not depend on how a prompt was cut into steps.  A column's key channels are
// dealt to `split` neighbouring lanes (channel d = lane_part * per_thread + i), each keeping its
// share of the column in registers; the dot with q is finished by shuffles.  The tokens' q, a, b
// and v come through shared memory in chunks, with the activations applied on the way in.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kScanThreads = 128;
constexpr int kChunk = 16;          // tokens staged at a time

__device__ __forceinline__ float scan_act(float z, int act) {
    return act == 1 ? z / (1.f + expf(-z)) : z;
}

template <typename T, int PER>
__global__ void __launch_bounds__(kScanThreads)
linear_scan_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                   int heads, int D, int V, int gate, const float* __restrict__ decay,
                   const float* __restrict__ f_bias, const float* __restrict__ floor_,
                   int q_act, int k_act, int v_act, float* __restrict__ state, int n_slots,
                   const int* __restrict__ q_start, const int* __restrict__ table_rows,
                   float* __restrict__ out, int split) {
    extern __shared__ float sh[];
    const int cols = kScanThreads / split;                  // value columns of this block
    float* q_sh = sh;                                       // [kChunk][D]
    float* a_sh = q_sh + kChunk * D;
    float* b_sh = a_sh + kChunk * D;
    float* v_sh = b_sh + kChunk * D;                        // [kChunk][cols]
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.z, h = blockIdx.y;
    const int col0 = blockIdx.x * cols;
    const int part = threadIdx.x % split, lc = threadIdx.x / split;
    const int col = col0 + lc;
    const int t0 = q_start[r], t1 = q_start[r + 1];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    const bool live = col < V;
    float* srow = state + (((size_t)slot * heads + h) * V + (live ? col : 0)) * D;
    const int d0 = part * PER;
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) S[i] = (live && d0 + i < D) ? srow[d0 + i] : 0.f;
    const float fixed = gate == 0 ? decay[h] : 0.f;

    for (int base = t0; base < t1; base += kChunk) {
        const int n = min(kChunk, t1 - base);
        __syncthreads();
        for (int i = threadIdx.x; i < n * D; i += kScanThreads) {
            const int j = i / D, d = i % D;
            const T* row = proj + (size_t)(base + j) * ld;
            q_sh[i] = scan_act(lsb_to_float(row[q_off + h * D + d]), q_act);
            const float z = lsb_to_float(row[k_off + h * D + d]);
            if (gate == 0) {
                a_sh[i] = fixed;
                b_sh[i] = scan_act(z, k_act);
            } else {
                const float lo = floor_[h * D + d];
                const float s = 1.f / (1.f + expf(-(z + (f_bias ? f_bias[h * D + d] : 0.f))));
                const float a = lo + (1.f - lo) * s;
                a_sh[i] = a;
                b_sh[i] = 1.f - a;
            }
        }
        for (int i = threadIdx.x; i < n * cols; i += kScanThreads) {
            const int j = i / cols, c = col0 + i % cols;
            v_sh[i] = c < V ? scan_act(lsb_to_float(proj[(size_t)(base + j) * ld + v_off + h * V + c]), v_act) : 0.f;
        }
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const float v = v_sh[j * cols + lc];
            const float* qj = q_sh + j * D + d0;
            const float* aj = a_sh + j * D + d0;
            const float* bj = b_sh + j * D + d0;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                if (d0 + i < D) {
                    S[i] = aj[i] * S[i] + bj[i] * v;
                    acc += S[i] * qj[i];
                }
            }
            for (int o = split >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (part == 0 && live) out[(size_t)(base + j) * heads * V + h * V + col] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (d0 + i < D) srow[d0 + i] = S[i];
    }
}

// The split of a column's channels over lanes (a power of two up to 32) and the channels a lane keeps.
static inline void scan_shape(int D, int* split, int* per) {
    int p = D <= 16 * 32 ? 16 : 32;
    if (D <= 8) p = 8;
    int s = 1;
    while (s < 32 && s * p < D) s <<= 1;
    *split = s;
    *per = p;
}

LSB_API int lsb_linear_scan_supported(int D) { return D > 0 && D <= 32 * 32; }

LSB_API int lsb_linear_scan(const void* proj, int dtype, long long ld, int q_off, int k_off, int v_off,
                            int heads, int D, int V, int gate, const float* decay, const float* f_bias,
                            const float* floor_, int q_act, int k_act, int v_act, float* state,
                            int n_slots, const int* q_start, const int* table_rows, int n_requests,
                            float* out, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || V <= 0 || !lsb_linear_scan_supported(D) || heads > 65535 || n_requests > 65535)
        return (int)cudaErrorInvalidValue;
    if ((gate == 0 && !decay) || (gate == 1 && !floor_) || gate < 0 || gate > 1) return (int)cudaErrorInvalidValue;
    int split, per;
    scan_shape(D, &split, &per);
    const int cols = kScanThreads / split;
    dim3 grid((V + cols - 1) / cols, heads, n_requests);
    const size_t smem = (size_t)kChunk * (3 * D + cols) * sizeof(float);
#define LSB_SCAN_LAUNCH(PER)                                                                          \
    do {                                                                                              \
        if (smem > 48 * 1024) {                                                                       \
            int rc = (int)cudaFuncSetAttribute(linear_scan_kernel<T, PER>,                            \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc) return rc;                                                                        \
        }                                                                                             \
        return lsb_launch(linear_scan_kernel<T, PER>, grid, dim3(kScanThreads), smem, stream, 1,      \
                          (const T*)proj, ld, q_off, k_off, v_off, heads, D, V, gate, decay, f_bias,  \
                          floor_, q_act, k_act, v_act, state, n_slots, q_start, table_rows, out, split); \
    } while (0)
    LSB_DISPATCH_DTYPE(dtype, {
        if (per == 8) LSB_SCAN_LAUNCH(8);
        else if (per == 16) LSB_SCAN_LAUNCH(16);
        else LSB_SCAN_LAUNCH(32);
    });
#undef LSB_SCAN_LAUNCH
    return 0;
}
