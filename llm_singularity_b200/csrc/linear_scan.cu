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
//   gate 2 (given):        a = keep[token, head] and b = write[token, head] * act_k(k projection), two
//                          numbers per token and head that another kernel has made (a memory
//                          whose gates are scalars per head); with `ones` a value column of ones
//                          rides along behind the V columns of the projection, so that the state
//                          has V + 1 columns and the last column of the output is (sum of b) . q
//   q = act_q(q projection) * q_scale, v = act_v(v projection); act: 0 none, 1 silu
//
// A block owns (request, head, a tile of value columns) and walks the request's tokens in order,
// so the result does not depend on how a prompt was cut into steps.  A column's key channels are
// dealt to `split` neighbouring lanes (channel d = lane_part * per_thread + i), each keeping its
// share of the column in registers; the dot with q is finished by shuffles.  The tokens' q, a, b
// and v come through shared memory in chunks of 16 tokens, with the activations applied on the way
// in; the projections' values of the next chunk are fetched (16-byte loads where the sizes allow)
// before the current chunk is walked, so the walk never waits for memory.
//
// Long portions are cut into segments that are walked side by side (MODE 1 - 3), since a walk is a
// chain of dependent steps and one portion alone gives each SM few of them: every segment is first
// walked from a zero state, which gives its own contribution E and the product P of its decays
// (MODE 1, no outputs); a small kernel then chains the segments, start(s + 1) = diag(P_s) start(s)
// + E_s, leaving each segment's start state and the request's new state; and every segment is
// walked again from its start state for the outputs (MODE 2).  Twice the arithmetic, a chain a
// segment long.  The sums form in another order than in one walk: equal beyond rounding.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kScanThreads = 128;
constexpr int kChunk = 16;          // tokens staged at a time

// 1 / (1 + e^-z).  Where the projections are bfloat16 their own rounding (2^-9) is five orders
// above that of the special-function unit's exponential and reciprocal, which cost a quarter of the
// exact ones; 32-bit storage keeps the exact functions.
template <typename T>
__device__ __forceinline__ float scan_sigmoid(float z) {
    if constexpr (sizeof(T) == 2) return __fdividef(1.f, 1.f + __expf(-z));
    else return 1.f / (1.f + expf(-z));
}
template <typename T>
__device__ __forceinline__ float scan_act(float z, int act) {
    return act == 1 ? z * scan_sigmoid<T>(z) : z;
}

// Raw projection values of one chunk, fetched a chunk ahead so that the loads are in flight while
// the chunk before is walked: up to kRawQ groups of eight channels of q and of k / f per thread,
// and kRawV groups of the block's value columns.
constexpr int kRawQ = 4, kRawV = 2;

template <typename T> struct alignas(16) ScanRaw { T q[kRawQ][8]; T k[kRawQ][8]; T v[kRawV][8]; };

template <typename T>
__device__ __forceinline__ void load8(T (&dst)[8], const T* src, bool vec) {
    if (vec) {
        if constexpr (sizeof(T) == 2) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        } else {
            *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
            *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
        }
    } else {
#pragma unroll
        for (int x = 0; x < 8; ++x) dst[x] = src[x];
    }
}

// Shared-memory place of channel d of a staged token: a lane's PER channels lie together, read as
// 16-byte vectors, and the shares of neighbouring lanes start PER + 4 words apart, which spreads
// the lanes of a quarter warp over all banks.
__device__ __forceinline__ int chan_slot(int d, int per, int) { return (d / per) * (per + 4) + d % per; }

template <typename T, int PER, int MODE>
__global__ void __launch_bounds__(kScanThreads)
linear_scan_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                   int heads, int D, int V, int gate, const float* __restrict__ decay,
                   const float* __restrict__ f_bias, const float* __restrict__ floor_,
                   int q_act, int k_act, int v_act, float* __restrict__ state, int n_slots,
                   const int* __restrict__ q_start, const int* __restrict__ table_rows,
                   float* __restrict__ out, int split, int vec, int seg_len, int max_segs,
                   float* __restrict__ seg_state, float* __restrict__ seg_decay,
                   const float* __restrict__ g_keep, const float* __restrict__ g_write, int ones, float q_scale) {
    extern __shared__ float sh[];
    const int cols = kScanThreads / split;                  // value columns of this block
    const int Dp = (PER + 4) * split;                       // a staged token's channels, with the padding
    float* q_sh = sh;                                       // [kChunk][Dp]
    float* a_sh = q_sh + kChunk * Dp;
    float* b_sh = a_sh + kChunk * Dp;
    float* v_sh = b_sh + kChunk * Dp;                       // [kChunk][cols]
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = MODE == 0 ? blockIdx.z : blockIdx.z / max_segs, h = blockIdx.y;
    const int sg = MODE == 0 ? 0 : blockIdx.z % max_segs;
    const int col0 = blockIdx.x * cols;
    const int part = threadIdx.x % split, lc = threadIdx.x / split;
    const int col = col0 + lc;
    int t0 = q_start[r], t1 = q_start[r + 1];
    if (MODE != 0) {
        t0 += sg * seg_len;
        t1 = min(t1, t0 + seg_len);
        if (t0 >= t1) return;                               // the request has fewer segments
    }
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    const int Vs = V + ones;                                // columns of the state and of the output
    const bool live = col < Vs;
    // where the walk starts from and where its end goes: the request's slot, or the segment's place
    float* srow = MODE == 0 ? state + (((size_t)slot * heads + h) * Vs + (live ? col : 0)) * D
                            : seg_state + ((((size_t)r * max_segs + sg) * heads + h) * Vs + (live ? col : 0)) * D;
    const int d0 = part * PER;
    float S[PER];
    float P[MODE == 1 ? PER : 1];
#pragma unroll
    for (int i = 0; i < PER; ++i) S[i] = (MODE != 1 && live && d0 + i < D) ? srow[d0 + i] : 0.f;
    if (MODE == 1) {
#pragma unroll
        for (int i = 0; i < (MODE == 1 ? PER : 1); ++i) P[i] = 1.f;
    }
    const float fixed = gate == 0 ? decay[h] : 0.f;

    // groups of eight consecutive channels (or value columns) of one staged token
    const int dg = (D + 7) / 8, vg = (cols + 7) / 8;
    const bool fits = kChunk * dg <= kRawQ * kScanThreads && kChunk * vg <= kRawV * kScanThreads;
    ScanRaw<T> raw;

    auto fetch = [&](int base, int n) {
#pragma unroll
        for (int u = 0; u < kRawQ; ++u) {
            const int g = threadIdx.x + u * kScanThreads;
            if (g < n * dg) {
                const int j = g / dg, d = (g % dg) * 8;
                const T* row = proj + (size_t)(base + j) * ld + h * D + d;
                const bool whole = vec && d + 8 <= D;
                if (whole || d + 8 <= D) {
                    if (MODE != 1) load8(raw.q[u], row + q_off, whole);      // (a segment's first walk makes no outputs)
                    load8(raw.k[u], row + k_off, whole);
                } else {
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        if (MODE != 1) raw.q[u][x] = d + x < D ? row[q_off + x] : lsb_from_float<T>(0.f);
                        raw.k[u][x] = d + x < D ? row[k_off + x] : lsb_from_float<T>(0.f);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kRawV; ++u) {
            const int g = threadIdx.x + u * kScanThreads;
            if (g < n * vg) {
                const int j = g / vg, c = (g % vg) * 8;
                const T* row = proj + (size_t)(base + j) * ld + v_off + h * V + col0 + c;
                const bool whole = vec && c + 8 <= cols && col0 + c + 8 <= V;
                if (whole) {
                    load8(raw.v[u], row, true);
                } else {
#pragma unroll
                    for (int x = 0; x < 8; ++x)
                        raw.v[u][x] = (c + x < cols && col0 + c + x < V) ? row[x] : lsb_from_float<T>(0.f);
                    // (the column of ones is put in when the chunk is staged)
                }
            }
        }
    };
    auto stage = [&](int base, int n) {
#pragma unroll
        for (int u = 0; u < kRawQ; ++u) {
            const int g = threadIdx.x + u * kScanThreads;
            if (g < n * dg) {
                const int j = g / dg, d = (g % dg) * 8;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    if (d + x >= D) break;
                    const int at = j * Dp + chan_slot(d + x, PER, split);
                    if (MODE != 1) q_sh[at] = scan_act<T>(lsb_to_float(raw.q[u][x]), q_act) * q_scale;
                    const float z = lsb_to_float(raw.k[u][x]);
                    if (gate == 0) {
                        a_sh[at] = fixed;
                        b_sh[at] = scan_act<T>(z, k_act);
                    } else if (gate == 2) {
                        a_sh[at] = g_keep[(size_t)(base + j) * heads + h];
                        b_sh[at] = g_write[(size_t)(base + j) * heads + h] * scan_act<T>(z, k_act);
                    } else {
                        const float lo = floor_[h * D + d + x];
                        const float sg = scan_sigmoid<T>(z + (f_bias ? f_bias[h * D + d + x] : 0.f));
                        const float a = lo + (1.f - lo) * sg;
                        a_sh[at] = a;
                        b_sh[at] = 1.f - a;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kRawV; ++u) {
            const int g = threadIdx.x + u * kScanThreads;
            if (g < n * vg) {
                const int j = g / vg, c = (g % vg) * 8;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    if (c + x < cols)
                        v_sh[j * cols + c + x] = (ones && col0 + c + x == V) ? 1.f
                                                                             : scan_act<T>(lsb_to_float(raw.v[u][x]), v_act);
            }
        }
    };
    // (sizes whose chunk does not fit the registers set aside above: plain loads, nothing ahead)
    auto stage_plain = [&](int base, int n) {
        for (int i = threadIdx.x; i < n * D; i += kScanThreads) {
            const int j = i / D, d = i % D;
            const T* row = proj + (size_t)(base + j) * ld;
            const int at = j * Dp + chan_slot(d, PER, split);
            if (MODE != 1) q_sh[at] = scan_act<T>(lsb_to_float(row[q_off + h * D + d]), q_act) * q_scale;
            const float z = lsb_to_float(row[k_off + h * D + d]);
            if (gate == 0) {
                a_sh[at] = fixed;
                b_sh[at] = scan_act<T>(z, k_act);
            } else if (gate == 2) {
                a_sh[at] = g_keep[(size_t)(base + j) * heads + h];
                b_sh[at] = g_write[(size_t)(base + j) * heads + h] * scan_act<T>(z, k_act);
            } else {
                const float lo = floor_[h * D + d];
                const float sg = scan_sigmoid<T>(z + (f_bias ? f_bias[h * D + d] : 0.f));
                const float a = lo + (1.f - lo) * sg;
                a_sh[at] = a;
                b_sh[at] = 1.f - a;
            }
        }
        for (int i = threadIdx.x; i < n * cols; i += kScanThreads) {
            const int j = i / cols, c = col0 + i % cols;
            v_sh[i] = c < V ? scan_act<T>(lsb_to_float(proj[(size_t)(base + j) * ld + v_off + h * V + c]), v_act)
                            : (ones && c == V) ? 1.f : 0.f;
        }
    };

    // channels past D (the last lane's share may reach beyond it) are staged as zeros once and
    // never written again: a = b = q = 0 keeps their state at zero, so the walk needs no bounds
    for (int i = threadIdx.x; i < 3 * kChunk * Dp; i += kScanThreads) sh[i] = 0.f;
    if (fits && t0 < t1) fetch(t0, min(kChunk, t1 - t0));
    const int mine = part * (PER + 4);
    for (int base = t0; base < t1; base += kChunk) {
        const int n = min(kChunk, t1 - base);
        __syncthreads();                                    // the chunk before has been walked
        if (fits) stage(base, n);
        else stage_plain(base, n);
        __syncthreads();
        if (fits && base + kChunk < t1) fetch(base + kChunk, min(kChunk, t1 - base - kChunk));
        // the walk: the next token's q, a and b are read (16-byte loads) while this one is worked on
        float4 qc[PER / 4], ac[PER / 4], bc[PER / 4];
#pragma unroll
        for (int x = 0; x < PER / 4; ++x) {
            qc[x] = *reinterpret_cast<const float4*>(q_sh + mine + 4 * x);
            ac[x] = *reinterpret_cast<const float4*>(a_sh + mine + 4 * x);
            bc[x] = *reinterpret_cast<const float4*>(b_sh + mine + 4 * x);
        }
        float vc = v_sh[lc];
#pragma unroll 2
        for (int j = 0; j < n; ++j) {
            float4 qn[PER / 4], an[PER / 4], bn[PER / 4];
            const int jn = j + 1 < n ? j + 1 : j;
#pragma unroll
            for (int x = 0; x < PER / 4; ++x) {
                qn[x] = *reinterpret_cast<const float4*>(q_sh + jn * Dp + mine + 4 * x);
                an[x] = *reinterpret_cast<const float4*>(a_sh + jn * Dp + mine + 4 * x);
                bn[x] = *reinterpret_cast<const float4*>(b_sh + jn * Dp + mine + 4 * x);
            }
            const float vn = v_sh[jn * cols + lc];
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int x = 0; x < PER / 4; ++x) {
                S[4 * x + 0] = ac[x].x * S[4 * x + 0] + bc[x].x * vc;
                S[4 * x + 1] = ac[x].y * S[4 * x + 1] + bc[x].y * vc;
                S[4 * x + 2] = ac[x].z * S[4 * x + 2] + bc[x].z * vc;
                S[4 * x + 3] = ac[x].w * S[4 * x + 3] + bc[x].w * vc;
                if (MODE != 1) {
                    acc0 += S[4 * x + 0] * qc[x].x;
                    acc1 += S[4 * x + 1] * qc[x].y;
                    acc0 += S[4 * x + 2] * qc[x].z;
                    acc1 += S[4 * x + 3] * qc[x].w;
                } else {
                    P[(MODE == 1 ? 4 * x : 0)] *= ac[x].x;
                    P[(MODE == 1 ? 4 * x + 1 : 0)] *= ac[x].y;
                    P[(MODE == 1 ? 4 * x + 2 : 0)] *= ac[x].z;
                    P[(MODE == 1 ? 4 * x + 3 : 0)] *= ac[x].w;
                }
            }
            if (MODE != 1) {
                float acc = acc0 + acc1;
                for (int o = split >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (part == 0 && live) out[(size_t)(base + j) * heads * Vs + h * Vs + col] = acc;
            }
#pragma unroll
            for (int x = 0; x < PER / 4; ++x) { qc[x] = qn[x]; ac[x] = an[x]; bc[x] = bn[x]; }
            vc = vn;
        }
    }
    if (MODE == 2) return;                                  // the chaining kernel has left the new state
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (d0 + i < D) srow[d0 + i] = S[i];
    }
    if (MODE == 1 && col0 == 0 && lc == 0) {                // the decays' product is the same for every column
        float* prow = seg_decay + (((size_t)r * max_segs + sg) * heads + h) * D;
#pragma unroll
        for (int i = 0; i < (MODE == 1 ? PER : 1); ++i)
            if (d0 + i < D) prow[d0 + i] = P[i];
    }
}

// start(0) = the slot's state; start(s + 1) = P_s * start(s) + E_s.  seg_state holds E_s coming in
// and start(s) going out; the slot gets the state after the last segment.
__global__ void scan_chain_kernel(float* __restrict__ state, int n_slots, float* __restrict__ seg_state,
                                  const float* __restrict__ seg_decay, const int* __restrict__ q_start,
                                  const int* __restrict__ table_rows, int heads, int D, int V, int seg_len,
                                  int max_segs) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.y;
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) return;
    const int n_segs = (q_start[r + 1] - q_start[r] + seg_len - 1) / seg_len;
    const size_t per = (size_t)heads * V * D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % D), h = (int)(i / ((size_t)V * D));
        float cur = state[(size_t)slot * per + i];
        for (int s0 = 0; s0 < n_segs; s0 += 8) {             // eight segments' loads in flight at once
            float e[8], p[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int s = s0 + k < n_segs ? s0 + k : n_segs - 1;
                e[k] = seg_state[((size_t)r * max_segs + s) * per + i];
                p[k] = seg_decay[(((size_t)r * max_segs + s) * heads + h) * D + d];
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (s0 + k < n_segs) {
                    seg_state[((size_t)r * max_segs + s0 + k) * per + i] = cur;
                    cur = p[k] * cur + e[k];
                }
            }
        }
        state[(size_t)slot * per + i] = cur;
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

// g_keep, g_write [tokens, heads]: gate 2 only.  ones: see above.  The state is [slots, heads, V + ones, D],
// out [tokens, heads, V + ones].
// seg_len > 0 with scratch given: portions longer than a segment are walked in segments side by
// side (see above); seg_state [requests * max_segs, heads, V, D] and seg_decay [requests * max_segs,
// heads, D] with max_segs = ceil(max_q_len / seg_len).
LSB_API int lsb_linear_scan(const void* proj, int dtype, long long ld, int q_off, int k_off, int v_off,
                            int heads, int D, int V, int gate, const float* decay, const float* f_bias,
                            const float* floor_, int q_act, int k_act, int v_act, float* state,
                            int n_slots, const int* q_start, const int* table_rows, int n_requests,
                            float* out, int seg_len, int max_q_len, float* seg_state, float* seg_decay,
                            const float* g_keep, const float* g_write, int ones, float q_scale,
                            cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || V <= 0 || !lsb_linear_scan_supported(D) || heads > 65535 || n_requests > 65535)
        return (int)cudaErrorInvalidValue;
    if ((gate == 0 && !decay) || (gate == 1 && !floor_) || (gate == 2 && (!g_keep || !g_write)) || gate < 0 || gate > 2)
        return (int)cudaErrorInvalidValue;
    ones = ones ? 1 : 0;
    const int Vs = V + ones;
    int split, per;
    scan_shape(D, &split, &per);
    const int cols = kScanThreads / split;
    const bool segmented = seg_len > 0 && seg_state && seg_decay && max_q_len > seg_len;
    const int max_segs = segmented ? (max_q_len + seg_len - 1) / seg_len : 1;
    if ((long long)n_requests * max_segs > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((Vs + cols - 1) / cols, heads, n_requests * max_segs);
    const size_t smem = (size_t)kChunk * (3 * (per + 4) * split + cols) * sizeof(float);
    // 16-byte loads of eight channels: every group of eight must start on a 16-byte boundary
    const int esz = dtype == LSB_F32 ? 4 : 2, al = 16 / esz;
    const int vec = ((uintptr_t)proj % 16 == 0 && ld % al == 0 && q_off % al == 0 && k_off % al == 0 &&
                     v_off % al == 0 && D % 8 == 0 && V % 8 == 0 && cols % 8 == 0) ? 1 : 0;
#define LSB_SCAN_LAUNCH(PER, MODE)                                                                    \
    do {                                                                                              \
        if (smem > 48 * 1024) {                                                                       \
            int rc = (int)cudaFuncSetAttribute(linear_scan_kernel<T, PER, MODE>,                      \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc) return rc;                                                                        \
        }                                                                                             \
        int rc = lsb_launch(linear_scan_kernel<T, PER, MODE>, grid, dim3(kScanThreads), smem, stream, 1, \
                          (const T*)proj, ld, q_off, k_off, v_off, heads, D, V, gate, decay, f_bias,  \
                          floor_, q_act, k_act, v_act, state, n_slots, q_start, table_rows, out, split, vec, \
                          seg_len, max_segs, seg_state, seg_decay, g_keep, g_write, ones, q_scale);   \
        if (rc) return rc;                                                                            \
    } while (0)
#define LSB_SCAN_PER(MODE)                                                                            \
    do {                                                                                              \
        if (per == 8) LSB_SCAN_LAUNCH(8, MODE);                                                       \
        else if (per == 16) LSB_SCAN_LAUNCH(16, MODE);                                                \
        else LSB_SCAN_LAUNCH(32, MODE);                                                               \
    } while (0)
    LSB_DISPATCH_DTYPE(dtype, {
        if (!segmented) {
            LSB_SCAN_PER(0);
        } else {
            LSB_SCAN_PER(1);
            const size_t per_state = (size_t)heads * Vs * D;
            const int blocks = (int)((per_state + 255) / 256 < 1024 ? (per_state + 255) / 256 : 1024);
            int rc = lsb_launch(scan_chain_kernel, dim3(blocks, n_requests), dim3(256), 0, stream, 1, state, n_slots,
                                seg_state, (const float*)seg_decay, q_start, table_rows, heads, D, Vs, seg_len, max_segs);
            if (rc) return rc;
            LSB_SCAN_PER(2);
        }
    });
#undef LSB_SCAN_PER
#undef LSB_SCAN_LAUNCH
    return 0;
}
