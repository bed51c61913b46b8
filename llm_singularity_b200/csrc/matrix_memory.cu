// The gates and the output step of a matrix memory with an exponential input gate (the mLSTM
// cell), around the walk of csrc/linear_scan.cu.  Per head and token, from the raw gate
// projections zi, zf (32-bit) and their biases:
//
//     i = cap * tanh((zi + bi) / cap)               f = logsigmoid(cap * tanh((zf + bf) / cap))
//     m_t = max(f + m_(t-1), i)                     (m starts at 0 when a request begins)
//     keep_t = exp(f + m_(t-1) - m_t)   write_t = exp(i - m_t)   floor_t = exp(-m_t)
//
// keep and write are what the walk multiplies the state and the incoming k v^T by (the same for
// every channel of the head); with a value column of ones riding along, the walk also carries the
// normaliser n and hands back n . q beside S^T q.  The output step then forms
//
//     o = S^T q / (max(|n . q|, floor_t) + 1e-6)
//     y = o / sqrt(mean(o^2) + eps) * w[head, :] * sigmoid(gate)         (mean over the head's values)
//
// The chain of maxima is walked in order, one warp per (request, head), with exactly the arithmetic
// above, while the transcendental functions on either side of it are spread over the lanes.
// Everything here is 32-bit.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kGatePer = 4;           // tokens a lane holds of a stretch of 128

__device__ __forceinline__ float mm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// raw [tokens, 2 * heads]: zi of every head, then zf.  gates [3][tokens][heads]: keep, write, floor.
// m_state [slots, heads].  One warp per (request, head): a lane holds four tokens of a stretch (token
// c * 32 + lane), their gates are formed side by side, the chain of maxima then runs through all 128
// in order on every lane alike (the values come by shuffle, which does not wait for the chain), and
// the projections of the next stretch are on their way meanwhile.
__global__ void __launch_bounds__(32)
memory_gates_kernel(const float* __restrict__ raw, const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                    float cap, float* __restrict__ m_state, int n_slots, const int* __restrict__ q_start,
                    const int* __restrict__ table_rows, float* __restrict__ gates, int tokens, int heads) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int h = blockIdx.x, r = blockIdx.y, lane = threadIdx.x;
    const int t0 = q_start[r], t1 = q_start[r + 1];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) {
        if (lane == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    float m = m_state[(size_t)slot * heads + h];
    const float bi = i_bias ? i_bias[h] : 0.f, bf = f_bias ? f_bias[h] : 0.f;
    const size_t plane = (size_t)tokens * heads;
    float zi[kGatePer], zf[kGatePer];
    auto fetch = [&](int base) {
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int t = base + c * 32 + lane;
            zi[c] = t < t1 ? raw[(size_t)t * 2 * heads + h] : 0.f;
            zf[c] = t < t1 ? raw[(size_t)t * 2 * heads + heads + h] : 0.f;
        }
    };
    fetch(t0);
    for (int base = t0; base < t1; base += 32 * kGatePer) {
        float gi[kGatePer], gf[kGatePer], before[kGatePer], now[kGatePer];
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            gi[c] = cap * tanhf((zi[c] + bi) / cap);
            gf[c] = mm_logsigmoid(cap * tanhf((zf[c] + bf) / cap));
            before[c] = now[c] = 0.f;
        }
        if (base + 32 * kGatePer < t1) fetch(base + 32 * kGatePer);
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int left = t1 - (base + c * 32);              // tokens of this group of 32 (the same on every lane)
            if (left <= 0) break;
            // (all 64 values are fetched before the chain starts: a shuffle issued between two steps of
            // the chain would make every step wait for it)
            float fv[32], iv[32];
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                fv[l] = __shfl_sync(0xffffffffu, gf[c], l);
                iv[l] = __shfl_sync(0xffffffffu, gi[c], l);
            }
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                if (l < left) {
                    const float prev = m;
                    m = fmaxf(fv[l] + m, iv[l]);
                    if (l == lane) {
                        before[c] = prev;
                        now[c] = m;
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int t = base + c * 32 + lane;
            if (t < t1) {
                const size_t at = (size_t)t * heads + h;
                gates[at] = expf(gf[c] + before[c] - now[c]);
                gates[plane + at] = expf(gi[c] - now[c]);
                gates[2 * plane + at] = expf(-now[c]);
            }
        }
    }
    if (lane == 0) m_state[(size_t)slot * heads + h] = m;
}

// Long portions: the same in three kernels, so that only the chain itself is walked by one warp per
// (request, head) and everything on either side of it is spread over the chip.
//   acts:  raw <- (i, f), in place, one thread per value
//   chain: gates <- (f + m_(t-1) - m_t, i - m_t, m_t), the maxima in order
//   exps:  gates <- (exp, exp, exp(-.)), in place
__global__ void __launch_bounds__(256)
memory_gate_acts_kernel(float* __restrict__ raw, const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                        float cap, int tokens, int heads) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const long long n = (long long)tokens * 2 * heads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % (2 * heads));
        const float z = raw[i];
        if (c < heads) raw[i] = cap * tanhf((z + (i_bias ? i_bias[c] : 0.f)) / cap);
        else raw[i] = mm_logsigmoid(cap * tanhf((z + (f_bias ? f_bias[c - heads] : 0.f)) / cap));
    }
}

__global__ void __launch_bounds__(32)
memory_gate_chain_kernel(const float* __restrict__ acts, float* __restrict__ m_state, int n_slots,
                         const int* __restrict__ q_start, const int* __restrict__ table_rows, float* __restrict__ gates,
                         int tokens, int heads) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int h = blockIdx.x, r = blockIdx.y, lane = threadIdx.x;
    const int t0 = q_start[r], t1 = q_start[r + 1];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) {
        if (lane == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    float m = m_state[(size_t)slot * heads + h];
    const size_t plane = (size_t)tokens * heads;
    float ni[kGatePer], nf[kGatePer];
    auto fetch = [&](int base) {
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int t = base + c * 32 + lane;
            ni[c] = t < t1 ? acts[(size_t)t * 2 * heads + h] : 0.f;
            nf[c] = t < t1 ? acts[(size_t)t * 2 * heads + heads + h] : 0.f;
        }
    };
    fetch(t0);
    for (int base = t0; base < t1; base += 32 * kGatePer) {
        float gi[kGatePer], gf[kGatePer], before[kGatePer], now[kGatePer];
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            gi[c] = ni[c];
            gf[c] = nf[c];
            before[c] = now[c] = 0.f;
        }
        if (base + 32 * kGatePer < t1) fetch(base + 32 * kGatePer);
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int left = t1 - (base + c * 32);
            if (left <= 0) break;
            // (all 64 values are fetched before the chain starts: a shuffle issued between two steps of
            // the chain would make every step wait for it)
            float fv[32], iv[32];
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                fv[l] = __shfl_sync(0xffffffffu, gf[c], l);
                iv[l] = __shfl_sync(0xffffffffu, gi[c], l);
            }
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                if (l < left) {
                    const float prev = m;
                    m = fmaxf(fv[l] + m, iv[l]);
                    if (l == lane) {
                        before[c] = prev;
                        now[c] = m;
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < kGatePer; ++c) {
            const int t = base + c * 32 + lane;
            if (t < t1) {
                const size_t at = (size_t)t * heads + h;
                gates[at] = gf[c] + before[c] - now[c];
                gates[plane + at] = gi[c] - now[c];
                gates[2 * plane + at] = now[c];
            }
        }
    }
    if (lane == 0) m_state[(size_t)slot * heads + h] = m;
}

__global__ void __launch_bounds__(256)
memory_gate_exps_kernel(float* __restrict__ gates, long long plane) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 3 * plane; i += (long long)gridDim.x * blockDim.x)
        gates[i] = expf(i < 2 * plane ? gates[i] : -gates[i]);
}

constexpr int kGatesApart = 256;      // portions from this many tokens on take the three kernels

// raw is overwritten where the three kernels run (a step whose longest portion has kGatesApart tokens or more).
LSB_API int lsb_memory_gates(float* raw, const float* i_bias, const float* f_bias, float cap, float* m_state,
                             int n_slots, const int* q_start, const int* table_rows, int n_requests, float* gates,
                             int tokens, int heads, int max_q_len, cudaStream_t stream) {
    if (n_requests <= 0 || tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || n_requests > 65535 || !(cap > 0.f)) return (int)cudaErrorInvalidValue;
    if (max_q_len >= kGatesApart) {
        const long long n = (long long)tokens * 2 * heads, plane = (long long)tokens * heads;
        int rc = lsb_launch(memory_gate_acts_kernel, dim3((unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096)),
                            dim3(256), 0, stream, 1, raw, i_bias, f_bias, cap, tokens, heads);
        if (rc) return rc;
        rc = lsb_launch(memory_gate_chain_kernel, dim3(heads, n_requests), dim3(32), 0, stream, 1, (const float*)raw,
                        m_state, n_slots, q_start, table_rows, gates, tokens, heads);
        if (rc) return rc;
        return lsb_launch(memory_gate_exps_kernel, dim3((unsigned)((3 * plane + 255) / 256 < 4096 ? (3 * plane + 255) / 256 : 4096)),
                          dim3(256), 0, stream, 1, gates, plane);
    }
    return lsb_launch(memory_gates_kernel, dim3(heads, n_requests), dim3(32), 0, stream, 1, (const float*)raw, i_bias, f_bias, cap,
                      m_state, n_slots, q_start, table_rows, gates, tokens, heads);
}

// walked [tokens, heads, V + 1]: S^T q in the first V columns of a head, n . q in the last.
// floor_ [tokens, heads].  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
memory_output_kernel(const float* __restrict__ walked, const float* __restrict__ floor_, const float* __restrict__ weight,
                     const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, int tokens, int heads, int V,
                     float eps) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const float* w = walked + (size_t)item * (V + 1);
    // one reciprocal for the row, and the row read once: a lane keeps up to kOutRegs of its values
    const float rden = 1.f / (fmaxf(fabsf(w[V]), floor_[item]) + 1e-6f);
    constexpr int kOutRegs = 8;
    float keep[kOutRegs];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kOutRegs; ++u) {
        const int c = lane + 32 * u;
        keep[u] = c < V ? w[c] * rden : 0.f;
        ss += keep[u] * keep[u];
    }
    for (int c = lane + 32 * kOutRegs; c < V; c += 32) {
        const float o = w[c] * rden;
        ss += o * o;
    }
    const float inv = rsqrtf(lsb_warp_sum(ss) / (float)V + eps);
    const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * V : nullptr;
    T* y = out + ((size_t)t * heads + h) * V;
#pragma unroll
    for (int u = 0; u < kOutRegs; ++u) {
        const int c = lane + 32 * u;
        if (c < V) {
            float v = keep[u] * inv * weight[h * V + c];
            if (g) v *= 1.f / (1.f + expf(-lsb_to_float(g[c])));
            y[c] = lsb_from_float<T>(v);
        }
    }
    for (int c = lane + 32 * kOutRegs; c < V; c += 32) {
        float v = w[c] * rden * inv * weight[h * V + c];
        if (g) v *= 1.f / (1.f + expf(-lsb_to_float(g[c])));
        y[c] = lsb_from_float<T>(v);
    }
}

LSB_API int lsb_memory_output(const float* walked, const float* floor_, const float* weight, const void* gate,
                              long long gate_stride, void* out, int dtype, int tokens, int heads, int V, float eps,
                              cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || V <= 0) return (int)cudaErrorInvalidValue;
    const long long items = (long long)tokens * heads;
    const int blocks = (int)((items + 3) / 4);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(memory_output_kernel<T>, dim3(blocks), dim3(128), 0, stream, 1, walked,
                                                floor_, weight, (const T*)gate, gate_stride, (T*)out, tokens, heads, V,
                                                eps));
    return 0;
}
