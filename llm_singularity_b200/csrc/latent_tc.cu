// Attention over a cached latent on the tensor cores (bfloat16 cache, warp-level MMA: mma.sync
// m16n8k16 fed by ldmatrix).
//
// Every head of a token reads the same cache rows (see latent.cu), so the (token, head) pairs of
// a request are the rows of one matrix: a block takes 64 of them, Q [64, kv_rank + rot_dim], and
// walks the request's keys in tiles of 64 rows of the cache.  Two warps share 16 rows: each makes
// S = Q K^T for its half of the tile's keys over the whole row width (accumulators in registers),
// they exchange their rows' maxima, and each writes the weights of its keys to shared memory; then
// each adds P V for its half of the first kv_rank columns of the same tile to its part of O
// (registers), which was rescaled by the change of the running maximum first.
//
// For steps of single tokens the keys of a request are split over `splits` blocks (grid.z), each
// writing a normalised partial result with its maximum and sum; a second kernel merges them.
//
// Scores, maxima, sums and weights are 32-bit; Q and P are rounded to bfloat16 as MMA operands.
#include "common.cuh"

#include <float.h>
#include <mma.h>

using namespace nvcuda;
typedef __nv_bfloat16 bf16;

LSB_DEFINE_STATUS()

constexpr int kRows = 64;               // (token, head) rows per block
constexpr int kKeys = 64;               // keys per tile
constexpr int kLtThreads = 256;         // 8 warps: 4 row groups x 2 column halves
constexpr int kMaxFrag = 16;            // 16-column fragments of O per warp: kv_rank <= 2 * 16 * 16
constexpr int kLdP = kKeys + 8;         // bfloat16 per row of the weight tile

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    // 16 bytes into shared memory without passing through registers; src_bytes 0 writes zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)),
                 "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Four 8 x 8 tiles of 16-bit values from shared memory, one row address per lane (lane i gives row
// i % 8 of tile i / 8); register j then holds tile j in the layout the MMA wants: lane t has the
// values (row t / 4, columns 2 (t % 4) and + 1), or with `trans` the same of the transposed tile.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// D (16 x 8, 32-bit) += A (16 x 16 bfloat16, rows) * B (16 x 8 bfloat16, columns)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int kMaxNt = 2 * kMaxFrag;    // 8-column tiles of O per warp

__global__ void __launch_bounds__(kLtThreads, 1)
latent_attention_tc_kernel(const float* __restrict__ qf, const bf16* __restrict__ pages,
                           const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                           const int* __restrict__ table_rows, const int* __restrict__ block_table,
                           int table_stride, bf16* __restrict__ out, float* __restrict__ part_o,
                           float* __restrict__ part_ml, int heads, int kv_rank, int rot_dim,
                           int page_size, int num_pages, float scale, int splits, int two) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int Dk = kv_rank + rot_dim, ldk = Dk + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem);                 // [64][ldk]
    bf16* Kbuf[2];                                            // [64][ldk] each; the second only if `two`
    Kbuf[0] = Qs + kRows * ldk;
    Kbuf[1] = Kbuf[0] + (two ? kKeys * ldk : 0);
    bf16* Ps = Kbuf[1] + kKeys * ldk;                         // [64][kLdP]: the tile's weights
    float* Mx = reinterpret_cast<float*>(Ps + kRows * kLdP);  // [2 halves][4 row groups][16 rows]
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.y, split = blockIdx.z;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int n_rows = q_len * heads;
    const int row0 = blockIdx.x * kRows;
    if (row0 >= n_rows) return;
    const int kv_len = kv_len_arr[r];
    const int first_pos = kv_len - q_len;
    const int last_row = min(row0 + kRows, n_rows) - 1;
    const int n_keys = first_pos + last_row / heads + 1;      // keys any row of this block may see
    int per = (n_keys + splits - 1) / splits;
    per = (per + kKeys - 1) / kKeys * kKeys;
    const int kbeg = split * per, kend = min(n_keys, kbeg + per);
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Q: rows of the block are consecutive rows of qf [(token, head), Dk]
    const float* qsrc = qf + ((size_t)qs * heads + row0) * Dk;
    for (int i = tid; i < kRows * Dk; i += kLtThreads) {
        const int row = i / Dk, d = i % Dk;
        Qs[row * ldk + d] = __float2bfloat16_rn(row0 + row < n_rows ? qsrc[(size_t)row * Dk + d] : 0.f);
    }
    // This lane's two rows of its warp's 16 (g and g + 8) and the last key each may see
    const int mi = warp & 3, half = warp >> 2;
    const int g = lane >> 2, tq = (lane & 3) * 2;             // row and column pair of a 16 x 8 result tile
    const int my_row[2] = {row0 + mi * 16 + g, row0 + mi * 16 + g + 8};
    int p_row[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) p_row[hr] = my_row[hr] < n_rows ? first_pos + my_row[hr] / heads : -1;
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};     // running maximum; sum over this warp's keys

    const int n_nt = kv_rank / 16;                            // 8-column tiles of O per warp (an even number)
    float acc[kMaxNt][4];
#pragma unroll
    for (int f = 0; f < kMaxNt; ++f) { acc[f][0] = acc[f][1] = acc[f][2] = acc[f][3] = 0.f; }
    // the rows and column offsets this lane gives to the tile loads (see ldsm_x4)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;      // A: 16 rows x 16 k
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;      // B from [n][k] rows

    // A tile of keys: four threads a cache row, every 16-byte piece an asynchronous copy of its
    // own, all in flight at once (rows past the last key are written as zeros).  With two buffers
    // the next tile is fetched while this one is worked on.
    const int chunks = Dk / 8;
    auto issue_tile = [&](int k0, bf16* dstK) {
        const int j = tid >> 2, kj = k0 + j;
        const bf16* src = pages;
        int bytes = 0;
        if (kj < kend) {
            const int page = bt[kj / page_size];
            if (page < 0 || page >= num_pages) lsb_set_status(LSB_BAD_PAGE);
            else { src = pages + ((size_t)page * page_size + kj % page_size) * Dk; bytes = 16; }
        }
        for (int c = tid & 3; c < chunks; c += 4)
            cp_async16(dstK + j * ldk + c * 8, bytes ? src + c * 8 : pages, bytes);
        cp_async_commit();
    };
    __syncthreads();                                          // Q is in place
    int buf = 0;
    if (kbeg < kend) issue_tile(kbeg, Kbuf[0]);
    for (int k0 = kbeg; k0 < kend; k0 += kKeys) {
        const bool more = k0 + kKeys < kend;
        if (two && more) {
            issue_tile(k0 + kKeys, Kbuf[buf ^ 1]);            // free since the barrier that ended the last tile
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        bf16* Ks = Kbuf[buf];
        // S = Q K^T: this warp's 16 rows x its 32 keys of the tile, four 16 x 8 result tiles
        float sacc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) { sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f; }
        {
            const bf16* qa = Qs + (mi * 16 + a_row) * ldk + a_col;
            const bf16* kb = Ks + (half * 32 + b_row) * ldk + b_col;
#pragma unroll 4
            for (int k = 0; k < Dk; k += 16) {
                uint32_t a[4], b01[4], b23[4];
                ldsm_x4(a, qa + k);
                ldsm_x4(b01, kb + k);                         // keys 0-15 of the warp's 32: (b0, b1) of two tiles
                ldsm_x4(b23, kb + 16 * ldk + k);              // keys 16-31
                mma_16816(sacc[0], a, b01[0], b01[1]);
                mma_16816(sacc[1], a, b01[2], b01[3]);
                mma_16816(sacc[2], a, b23[0], b23[1]);
                mma_16816(sacc[3], a, b23[2], b23[3]);
            }
        }
        // scale and mask; the maximum of each of the lane's rows over the warp's 32 keys
        float hmax[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kj = k0 + half * 32 + nt * 8 + tq + (e & 1), hr = e >> 1;
                const float v = (kj <= p_row[hr] && kj < kend) ? sacc[nt][e] * scale : -FLT_MAX;
                sacc[nt][e] = v;
                hmax[hr] = fmaxf(hmax[hr], v);
            }
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            hmax[hr] = fmaxf(hmax[hr], __shfl_xor_sync(0xffffffffu, hmax[hr], 1));
            hmax[hr] = fmaxf(hmax[hr], __shfl_xor_sync(0xffffffffu, hmax[hr], 2));
        }
        // the two warps that share 16 rows (one for each half of the keys) tell each other
        if ((lane & 3) == 0) {
            Mx[(half * 4 + mi) * 16 + g] = hmax[0];
            Mx[(half * 4 + mi) * 16 + g + 8] = hmax[1];
        }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const float other = Mx[((half ^ 1) * 4 + mi) * 16 + g + 8 * hr];
            const float m_new = fmaxf(m[hr], fmaxf(hmax[hr], other));
            corr[hr] = expf(m[hr] - m_new);                   // both -FLT_MAX at first: 1, on sums that are 0
            m[hr] = m_new;
        }
        // weights of the warp's 32 keys -> shared memory (bfloat16), their sums into l
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = sacc[nt][e] > -FLT_MAX ? expf(sacc[nt][e] - m[e >> 1]) : 0.f;
                psum[e >> 1] += p[e];
            }
            bf16* dst = Ps + (mi * 16 + g) * kLdP + half * 32 + nt * 8 + tq;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(p[0], p[1]);
            *reinterpret_cast<__nv_bfloat162*>(dst + 8 * kLdP) = __floats2bfloat162_rn(p[2], p[3]);
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            psum[hr] += __shfl_xor_sync(0xffffffffu, psum[hr], 1);
            psum[hr] += __shfl_xor_sync(0xffffffffu, psum[hr], 2);
            l[hr] = l[hr] * corr[hr] + psum[hr];
        }
        // what O holds was weighted against the old maximum
#pragma unroll
        for (int f = 0; f < kMaxNt; ++f) {
            if (f < n_nt) {
                acc[f][0] *= corr[0]; acc[f][1] *= corr[0];
                acc[f][2] *= corr[1]; acc[f][3] *= corr[1];
            }
        }
        __syncthreads();                                      // all 64 keys' weights are in place
        {
            // O += P V: this warp's 16 rows x its half of the value columns.  V is the tile of keys
            // itself, [key][dim]: its 8 x 8 pieces are transposed on the way into the registers.
            const bf16* pa = Ps + (mi * 16 + a_row) * kLdP + a_col;
            const bf16* vb = Ks + a_row * ldk + half * (kv_rank / 2) + a_col;
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk) {
                uint32_t a[4];
                ldsm_x4(a, pa + kk * 16);
#pragma unroll
                for (int f = 0; f < kMaxNt; f += 2) {
                    if (f < n_nt) {
                        uint32_t b[4];                        // (b0, b1) of column tile f, then of f + 1
                        ldsm_x4_trans(b, vb + kk * 16 * ldk + f * 8);
                        mma_16816(acc[f], a, b[0], b[1]);
                        mma_16816(acc[f + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                      // this tile and its weights are done with
        if (two) buf ^= 1;
        else if (more) issue_tile(k0 + kKeys, Kbuf[0]);
    }
    // a row's sum is the two halves' sums (they were kept against the same maxima)
    if ((lane & 3) == 0) {
        Mx[(half * 4 + mi) * 16 + g] = l[0];
        Mx[(half * 4 + mi) * 16 + g + 8] = l[1];
    }
    __syncthreads();
    float inv_l[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        l[hr] += Mx[((half ^ 1) * 4 + mi) * 16 + g + 8 * hr];
        inv_l[hr] = l[hr] > 0.f ? 1.f / l[hr] : 0.f;
    }
    if (splits > 1 && half == 0 && (lane & 3) == 0) {
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            if (my_row[hr] < n_rows) {
                float* ml = part_ml + (((size_t)qs * heads + my_row[hr]) * splits + split) * 2;
                ml[0] = m[hr];
                ml[1] = l[hr];
            }
        }
    }
#pragma unroll
    for (int f = 0; f < kMaxNt; ++f) {
        if (f < n_nt) {
            const int col = half * (kv_rank / 2) + f * 8 + tq;
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {                  // rows g and g + 8 of the warp's 16
                const int grow = my_row[hr];
                if (grow >= n_rows) continue;
                const float v0 = acc[f][2 * hr] * inv_l[hr], v1 = acc[f][2 * hr + 1] * inv_l[hr];
                if (splits > 1) {
                    float* dst = part_o + (((size_t)qs * heads + grow) * splits + split) * kv_rank + col;
                    *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
                } else {
                    bf16* dst = out + ((size_t)qs * heads + grow) * kv_rank + col;
                    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
                }
            }
        }
    }
}

// out[row] = sum over splits of w_s part_o[row, s], w_s = l_s e^(m_s - M) / sum of the same
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int splits, int kv_rank) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * splits * 2;
    float M = -FLT_MAX;
    for (int s = 0; s < splits; ++s)
        if (ml[2 * s + 1] > 0.f) M = fmaxf(M, ml[2 * s]);
    float total = 0.f;
    for (int s = 0; s < splits; ++s)
        if (ml[2 * s + 1] > 0.f) total += ml[2 * s + 1] * expf(ml[2 * s] - M);
    const float inv = total > 0.f ? 1.f / total : 0.f;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ls = ml[2 * s + 1];
            if (ls > 0.f) acc += ls * expf(ml[2 * s] - M) * inv * part_o[(row * splits + s) * kv_rank + d];
        }
        out[row * kv_rank + d] = __float2bfloat16_rn(acc);
    }
}

static size_t latent_tc_smem(int kv_rank, int rot_dim, int key_buffers = 1) {
    const size_t ldk = kv_rank + rot_dim + 8;
    return (1 + key_buffers) * kRows * ldk * sizeof(bf16) + kRows * kLdP * sizeof(bf16) + 128 * sizeof(float);
}

LSB_API int lsb_latent_attention_tc_supported(int kv_rank, int rot_dim) {
    return kv_rank > 0 && kv_rank % 32 == 0 && kv_rank <= 32 * kMaxFrag && rot_dim >= 0 && rot_dim % 16 == 0 &&
           latent_tc_smem(kv_rank, rot_dim) <= 200 * 1024;
}

// part_o [tokens * heads, splits, kv_rank] and part_ml [tokens * heads, splits, 2] are needed when
// splits > 1 (steps of single tokens); out [tokens, heads, kv_rank] bfloat16.
LSB_API int lsb_latent_attention_tc(const float* qf, const void* pages, const int* q_start, const int* kv_len,
                                    const int* table_rows, const int* block_table, int table_stride,
                                    void* out, float* part_o, float* part_ml, int n_requests, int max_q_len,
                                    int n_tokens, int heads, int kv_rank, int rot_dim, int page_size,
                                    int num_pages, float scale, int splits, cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (!lsb_latent_attention_tc_supported(kv_rank, rot_dim) || heads <= 0 || n_requests > 65535 || splits < 1 ||
        splits > 65535 || (splits > 1 && (!part_o || !part_ml)))
        return (int)cudaErrorInvalidValue;
    static int configured = -1;
    const int two = latent_tc_smem(kv_rank, rot_dim, 2) <= 200 * 1024 ? 1 : 0;
    const size_t smem = latent_tc_smem(kv_rank, rot_dim, 1 + two);
    if (configured < 0)
        configured = (int)cudaFuncSetAttribute(latent_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               200 * 1024);
    if (configured) return configured;
    const long long rows = (long long)max_q_len * heads;
    dim3 grid((unsigned)((rows + kRows - 1) / kRows), n_requests, splits);
    int rc = lsb_launch(latent_attention_tc_kernel, grid, dim3(kLtThreads), smem, stream, 1, qf, (const bf16*)pages,
                        q_start, kv_len, table_rows, block_table, table_stride, (bf16*)out, part_o, part_ml, heads,
                        kv_rank, rot_dim, page_size, num_pages, scale, splits, two);
    if (rc || splits == 1) return rc;
    return lsb_launch(latent_merge_kernel, dim3((unsigned)((long long)n_tokens * heads)), dim3(128), 0, stream, 1,
                      (const float*)part_o, (const float*)part_ml, (bf16*)out, splits, kv_rank);
}

// ------------------------------------------------------------------ per-head products
// C[m, h, :] = A[m, h, :] B[h]^T for every head h on warp-level MMA: A (32-bit or bfloat16, rounded
// to bfloat16 as an operand) with any row and head strides, B [heads, N, K] bfloat16, C 32-bit or
// bfloat16 with any row and head strides; 32-bit accumulation.  A block makes a 64 x 64 tile of
// one head, K in slabs of 32 staged through shared memory (so no size needs to be a multiple of
// anything); four warps, 32 x 32 each.
constexpr int kBtT = 64, kBtK = 32, kBtLd = kBtK + 8;

template <typename TA, typename TC>
__global__ void __launch_bounds__(128)
batched_nt_tc_kernel(const TA* __restrict__ A, long long lda, long long a_bs, const bf16* __restrict__ B,
                     TC* __restrict__ C, long long ldc, long long c_bs, int M, int N, int K, int vec_a, int vec_b) {
    __shared__ __align__(32) bf16 As[kBtT * kBtLd];
    __shared__ __align__(32) bf16 Bs[kBtT * kBtLd];
    __shared__ __align__(32) float stage_all[4 * 256];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int h = blockIdx.z, m0 = blockIdx.y * kBtT, n0 = blockIdx.x * kBtT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 1, wn = warp >> 1;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[i][j], 0.f);
    for (int k0 = 0; k0 < K; k0 += kBtK) {
        // a slab of 64 rows x 32 k of each operand: 16-byte pieces where the addresses allow (the
        // two pieces a thread fetches of each operand are independent loads), single values else
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int piece = tid + u * 128;                  // 256 pieces of 8 values
            const int row = piece >> 2, col = (piece & 3) * 8;
            const int k = k0 + col, m = m0 + row, n = n0 + row;
            bf16* da = As + row * kBtLd + col;
            bf16* db = Bs + row * kBtLd + col;
            if (vec_b && n < N && k + 8 <= K) {
                *reinterpret_cast<uint4*>(db) = *reinterpret_cast<const uint4*>(B + ((size_t)h * N + n) * K + k);
            } else {
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    db[x] = (n < N && k + x < K) ? B[((size_t)h * N + n) * K + k + x] : __float2bfloat16_rn(0.f);
            }
            const TA* pa = A + (size_t)m * lda + (size_t)h * a_bs + k;
            if (vec_a && m < M && k + 8 <= K) {
                if constexpr (sizeof(TA) == 2) {
                    *reinterpret_cast<uint4*>(da) = *reinterpret_cast<const uint4*>(pa);
                } else {
                    const float4 lo = *reinterpret_cast<const float4*>(pa), hi = *reinterpret_cast<const float4*>(pa + 4);
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
                    *reinterpret_cast<uint4*>(da) = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                                               *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
                }
            } else {
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    da[x] = (m < M && k + x < K) ? __float2bfloat16_rn(lsb_to_float(pa[x])) : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBtK; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a[2];
            wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                wmma::load_matrix_sync(a[i], As + (wm * 32 + i * 16) * kBtLd + kk, kBtLd);
                wmma::load_matrix_sync(b[i], Bs + (wn * 32 + i * 16) * kBtLd + kk, kBtLd);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) wmma::mma_sync(acc[i][j], a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* stage = stage_all + warp * 256;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            wmma::store_matrix_sync(stage, acc[i][j], 16, wmma::mem_row_major);
            __syncwarp();
            const int row = lane >> 1, c0 = (lane & 1) * 8;
            const int m = m0 + wm * 32 + i * 16 + row;
            if (m < M) {
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const int n = n0 + wn * 32 + j * 16 + c0 + x;
                    if (n < N) C[(size_t)m * ldc + (size_t)h * c_bs + n] = lsb_from_float<TC>(stage[row * 16 + c0 + x]);
                }
            }
            __syncwarp();
        }
    }
}

// ta / tc: 0 = 32-bit, 1 = bfloat16 (A and C); B is bfloat16
LSB_API int lsb_batched_nt_tc(const void* A, int ta, long long lda, long long a_bs, const void* B, void* C, int tc,
                              long long ldc, long long c_bs, int M, int N, int K, int batch, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || batch > 65535 || (M + kBtT - 1) / kBtT > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + kBtT - 1) / kBtT, (M + kBtT - 1) / kBtT, batch);
    // 16-byte loads: every piece of eight values must start on a 16-byte (A in 32-bit: 32-byte) boundary
    const int ea = ta == 0 ? 4 : 2;
    const int vec_a = ((uintptr_t)A % (8 * ea) == 0 && (lda * ea) % (8 * ea) == 0 && (a_bs * ea) % (8 * ea) == 0) ? 1 : 0;
    const int vec_b = ((uintptr_t)B % 16 == 0 && K % 8 == 0) ? 1 : 0;
#define LSB_BNT(TA, TC)                                                                              \
    return lsb_launch(batched_nt_tc_kernel<TA, TC>, grid, dim3(128), 0, stream, 1, (const TA*)A, lda, a_bs, \
                      (const bf16*)B, (TC*)C, ldc, c_bs, M, N, K, vec_a, vec_b)
    if (ta == 0 && tc == 0) LSB_BNT(float, float);
    if (ta == 0 && tc == 1) LSB_BNT(float, bf16);
    if (ta == 1 && tc == 0) LSB_BNT(bf16, float);
    if (ta == 1 && tc == 1) LSB_BNT(bf16, bf16);
#undef LSB_BNT
    return (int)cudaErrorInvalidValue;
}
