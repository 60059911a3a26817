// K2: W4A16 GEMV / skinny GEMM (batch tile of 8 rows of X), HBM-bound.
//
// Y[M,N] = X[M,K] . W^T with W dequantised in registers and never written to memory.
//
// Work split
//   grid.x : blocks of 64 output columns (4 warps x 16 weight rows)
//   grid.y : K splits (split-K); partial sums meet in caller-provided fp32 scratch, the last
//            block to arrive for a column block sums them in split order (deterministic)
//   grid.z : batch tiles of 8 rows of X
// Weight stream: every lane copies 16 B (32 codes) of weight row g = lane/4 and of row g+8 per
// 128-code chunk of K with cp.async.cg (L2 -> shared memory, no registers, no L1) into a ring that is
// PRIVATE to the lane, GEMV_DEPTH chunks deep; a lane reads back only what it copied itself, so the
// stream needs no block-level synchronisation. The 4 lanes of a row cover 64 contiguous bytes and
// the ring keeps 512 contiguous bytes per row in flight.
// Per block, once: the (row, group) constants of the converter (magic+zero, duplicated scale) are
// computed into a shared table, and the activations are staged in the order the converter produces
// code pairs, (c_i, c_{i+4}) -- the contraction index may be permuted freely as long as A and B
// agree -- so no per-weight shuffle is spent on ordering.
// Per warp and chunk: 2 x 16 B of codes -> lop3 / packed 16-bit arithmetic -> A fragments of eight
// m16n8k16 tensor-core MMAs whose B fragments are the staged activations; fp32 accumulation.
#include <mutex>

#include "qf_common.cuh"

namespace qf {

constexpr int GEMV_THREADS = 128;
constexpr int GEMV_WARPS = 4;
constexpr int GEMV_ROWS_PER_BLOCK = 16 * GEMV_WARPS;  // 64
constexpr int GEMV_DEPTH = 8;                         // chunks in flight per lane
constexpr int GEMV_MAX_CHUNKS_PER_SPLIT = 32;
constexpr int GEMV_RING_BYTES = GEMV_DEPTH * 2 * GEMV_THREADS * 16;  // 32 KB

struct GemvParams {
    const uint16_t *X;
    const uint32_t *qw;
    const uint16_t *scales;
    const void *zeros;
    void *Y;
    float *partial;     // [split_k][m_tiles*8][N]
    int *counters;      // [col_blocks * m_tiles], zero between launches
    int64_t M, N, K;
    int group_chunks;   // group_size / 128
    int chunks;         // K / 128
    int chunks_per_split;
    int split_k;
    int out_dtype;
    int zero_const;
    int m_pad;          // rows of X staged per batch tile: 1, 2, 4 or 8
    int cluster_reduce; // 1: the split_k blocks of a column block form a thread-block cluster (rank = split) and
                        //    sum their partial outputs through distributed shared memory
};

// dynamic shared memory: ring | constants table [chunks][64 rows] uint2 | staged X [chunks][4][m_pad][4] uint4
static inline size_t gemv_smem_bytes(int chunks_per_split, int m_pad) {
    return (size_t)GEMV_RING_BYTES + (size_t)chunks_per_split * GEMV_ROWS_PER_BLOCK * 8 +
           (size_t)chunks_per_split * 4 * m_pad * 4 * 16;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Converter constants from a table entry (x = magic+zero duplicated, y = scale duplicated).
template <bool BF16>
__device__ __forceinline__ ZeroScale<BF16> consts_from(const uint2 e) {
    ZeroScale<BF16> zs;
    zs.zsub = e.x;
    zs.s2 = e.y;
    // f16 only: -(64 + z) = (1024 + z) * (-1) + 960, exact in f16
    zs.zfma = BF16 ? 0u : fma_f16x2(e.x, 0xbc00bc00u, 0x63806380u);
    return zs;
}

// MPAD: rows of X staged per batch tile (1, 2, 4 or 8), a compile-time constant so that the activation
// addressing in the main loop folds into immediates.
// AR: this GPU holds a K shard of the weights (row-parallel linear). The block that finishes a column block
// pushes its 64 x M fp32 partial outputs into every rank's slot with peer stores, each value paired with the
// call's token in one 8-byte store, then polls (bounded) its own slots until every rank's pair for the same
// element carries that token, sums in rank order (same bits on every rank) and writes Y. The exchange of a
// column block overlaps the weight streams of the blocks still running; no separate all-reduce kernel follows.
// A waiting block depends only on blocks that the peers dispatched before their own waiting blocks (blocks are
// dispatched in index order and a block waits only after every block of its column has arrived), so waiters
// cannot starve the work they wait for; the wait is bounded all the same.
template <bool BF16, int ZMODE, int MPAD, bool AR>
__device__ __forceinline__ void gemv_body(const GemvParams &p, const typename ExchArg<AR>::type &ar) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ int s_is_last;
    __shared__ volatile int s_ar_fail;
    __shared__ float s_tile[8 * GEMV_ROWS_PER_BLOCK];  // [batch row][column]: this block's partial or finished outputs

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int split = blockIdx.y;
    const int mt = blockIdx.z;
    const int c0 = split * p.chunks_per_split;
    const int c1 = min(c0 + p.chunks_per_split, p.chunks);
    const int nch = c1 - c0;
    const int64_t n_blk = (int64_t)blockIdx.x * GEMV_ROWS_PER_BLOCK;
    const int64_t row_a = n_blk + warp * 16 + g;
    const bool warp_active = (n_blk + warp * 16) < p.N;  // N is a multiple of 16
    constexpr int m_pad = MPAD;

    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_raw) + (uint32_t)tid * 16u;  // + slot * 2048
    const uint32_t table = (uint32_t)__cvta_generic_to_shared(smem_raw) + GEMV_RING_BYTES;     // [chunk][64] uint2
    const uint32_t xs = table + (uint32_t)p.chunks_per_split * GEMV_ROWS_PER_BLOCK * 8u;       // [chunk][4][m_pad][4]

    // 1. weight stream: fill the ring before anything else
    const uint32_t *ra = p.qw + row_a * (p.K >> 3) + (int64_t)c0 * 16 + t * 4;
    const uint32_t *rb = ra + 8 * (p.K >> 3);
#pragma unroll
    for (int i = 0; i < GEMV_DEPTH; ++i) {
        if (warp_active && i < nch) {
            cp_async16(ring + (uint32_t)(2 * i) * 2048u, ra + i * 16);
            cp_async16(ring + (uint32_t)(2 * i + 1) * 2048u, rb + i * 16);
        }
        cp_async_commit();
    }

    // 2. converter constants of this block's (chunk, row) pairs
    for (int e = tid; e < nch * GEMV_ROWS_PER_BLOCK; e += GEMV_THREADS) {
        const int r = e & (GEMV_ROWS_PER_BLOCK - 1);
        const int cl = e >> 6;
        const int64_t n = n_blk + r;
        uint2 ent = make_uint2(0u, 0u);
        if (n < p.N) {
            const int64_t gi = p.group_chunks == 1 ? (c0 + cl) : (c0 + cl) / p.group_chunks;
            ZeroScale<BF16> zs;
            zs.set(load_zero<ZMODE>(p.zeros, p.zero_const, gi, n, p.N), __ldg(p.scales + gi * p.N + n));
            ent = make_uint2(zs.zsub, zs.s2);
        }
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(table + (uint32_t)e * 8u), "r"(ent.x), "r"(ent.y));
    }

    // Everything above is independent of the previous kernel in the stream; the activations are not.
    griddep_launch_dependents();
    griddep_wait();
    unsigned ar_epoch = 0;
    if constexpr (AR) ar_epoch = exch_read_epoch(ar);

    // 3. activations of this K range in fragment order, zero rows beyond M
    {
        const int units_per_chunk = m_pad * 16;  // 16-byte pieces: (m) x (t*4 + j)
        const int64_t m_base = (int64_t)mt * 8;
        for (int u = tid; u < nch * units_per_chunk; u += GEMV_THREADS) {
            const int piece = u & 15;  // = t*4 + j : 16-byte piece of the chunk's 256-byte row segment
            const int m = (u >> 4) % m_pad;
            const int cl = u / units_per_chunk;
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (m_base + m < p.M) {
                const uint4 v = *reinterpret_cast<const uint4 *>(p.X + (m_base + m) * p.K + (int64_t)(c0 + cl) * 128 +
                                                                 piece * 8);
                r.x = prmt(v.x, v.z, 0x5410u);  // (e0, e4)
                r.y = prmt(v.x, v.z, 0x7632u);  // (e1, e5)
                r.z = prmt(v.y, v.w, 0x5410u);  // (e2, e6)
                r.w = prmt(v.y, v.w, 0x7632u);  // (e3, e7)
            }
            const int tt = piece >> 2, j = piece & 3;
            const uint32_t dst = xs + (uint32_t)((((cl * 4 + j) * m_pad + m) * 4 + tt) * 16);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w));
        }
    }
    __syncthreads();

    // 4. main loop: wait for the oldest chunk of the ring, read it back, refill its slot, convert, MMA
    float acc2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // two chains: MMAs of one chain are dependent
    if (warp_active) {
        // Batch columns >= m_pad of the MMA are never stored, so their lanes may read any staged row:
        // wrap g into the staged rows instead of zero-filling registers.
        uint32_t xc = xs + (uint32_t)(((g & (m_pad - 1)) * 4 + t) * 16);
        uint32_t tab = table + (uint32_t)(warp * 16 + g) * 8u;
        const uint32_t *ga = ra + GEMV_DEPTH * 16;  // next chunk to request
        const uint32_t *gb = rb + GEMV_DEPTH * 16;
#pragma unroll 1
        for (int i = 0; i < nch; ++i) {
            cp_async_wait<GEMV_DEPTH - 1>();
            const uint32_t slot = ring + ((uint32_t)(i & (GEMV_DEPTH - 1)) << 12);
            const uint4 va = lds128g(slot);
            const uint4 vb = lds128g(slot + 2048u);
            if (i + GEMV_DEPTH < nch) {
                cp_async16(slot, ga);
                cp_async16(slot + 2048u, gb);
            }
            cp_async_commit();
            ga += 16;
            gb += 16;
            const ZeroScale<BF16> za = consts_from<BF16>(lds64g(tab));
            const ZeroScale<BF16> zb = consts_from<BF16>(lds64g(tab + 64u));
            const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
            const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t pa[4], pb[4];
                dequant8<BF16>(wa[j], za, pa);
                dequant8<BF16>(wb[j], zb, pb);
                const uint4 xb = lds128g(xc + (uint32_t)(j * m_pad * 64));
                mma_16816<BF16>(acc2[0], pa[0], pb[0], pa[1], pb[1], xb.x, xb.y);
                mma_16816<BF16>(acc2[1], pa[2], pb[2], pa[3], pb[3], xb.z, xb.w);
            }
            tab += GEMV_ROWS_PER_BLOCK * 8u;
            xc += 4u * m_pad * 64u;
        }
    }
    cp_async_wait<0>();

    // 5. epilogue. acc[0..1]: row g, batch 2t, 2t+1 ; acc[2..3]: row g+8
    float acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = acc2[0][i] + acc2[1][i];
    const int64_t m0 = (int64_t)mt * 8 + 2 * t;
    if (!AR && p.split_k == 1) {
        if (warp_active) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (m0 + e < p.M) {
                    store_out(p.Y, p.out_dtype, (m0 + e) * p.N + row_a, acc[e]);
                    store_out(p.Y, p.out_dtype, (m0 + e) * p.N + row_a + 8, acc[2 + e]);
                }
            }
        }
        return;
    }

    const int m_rows = min(8, m_pad + (m_pad & 1));  // rows of this batch tile that hold partial sums
    if (!AR && p.cluster_reduce) {
        // Split-K inside a cluster: every block leaves its partial outputs in its own shared memory, the cluster
        // meets, and each block sums its share of the column block from all blocks in split order.
        if (warp_active && 2 * t < m_pad) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s_tile[(2 * t + e) * GEMV_ROWS_PER_BLOCK + warp * 16 + g] = acc[e];
                s_tile[(2 * t + e) * GEMV_ROWS_PER_BLOCK + warp * 16 + g + 8] = acc[2 + e];
            }
        }
        cluster_sync_all();
        const int units = GEMV_ROWS_PER_BLOCK * m_rows;
        const int per = (units + p.split_k - 1) / p.split_k;
        const int u_end = min(units, (split + 1) * per);
        const uint32_t tile = (uint32_t)__cvta_generic_to_shared(s_tile);
        for (int u = split * per + tid; u < u_end; u += GEMV_THREADS) {
            const int64_t n = n_blk + (u & (GEMV_ROWS_PER_BLOCK - 1));
            const int64_t mm = (int64_t)mt * 8 + u / GEMV_ROWS_PER_BLOCK;
            if (n < p.N && mm < p.M) {
                float v[8];
#pragma unroll
                for (int sp = 0; sp < 8; ++sp)
                    v[sp] = sp < p.split_k ? ld_dsmem_f1(dsmem_addr(tile + 4u * (uint32_t)u, (uint32_t)sp)) : 0.f;
                float s = 0.f;
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) s += v[sp];
                store_out(p.Y, p.out_dtype, mm * p.N + n, s);
            }
        }
        cluster_sync_all();  // nobody leaves while its partial outputs may still be read
        return;
    }
    if (AR && p.split_k == 1) {
        if (warp_active && 2 * t < m_pad) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s_tile[(2 * t + e) * GEMV_ROWS_PER_BLOCK + warp * 16 + g] = acc[e];
                s_tile[(2 * t + e) * GEMV_ROWS_PER_BLOCK + warp * 16 + g + 8] = acc[2 + e];
            }
        }
        __syncthreads();
    } else {
        const int64_t Mp = (int64_t)gridDim.z * 8;
        if (warp_active && 2 * t < m_pad) {
            float *dst = p.partial + ((int64_t)split * Mp + m0) * p.N;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                __stcg(dst + e * p.N + row_a, acc[e]);
                __stcg(dst + e * p.N + row_a + 8, acc[2 + e]);
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int *cnt = p.counters + blockIdx.z * gridDim.x + blockIdx.x;
            const int prev = atomicAdd(cnt, 1);
            s_is_last = (prev == p.split_k - 1);
            if (s_is_last) *cnt = 0;  // ready for the next launch
        }
        __syncthreads();
        if (!s_is_last) return;
        __threadfence();
        for (int u = tid; u < GEMV_ROWS_PER_BLOCK * m_rows; u += GEMV_THREADS) {
            const int nl = u & (GEMV_ROWS_PER_BLOCK - 1);
            const int m = u / GEMV_ROWS_PER_BLOCK;
            const int64_t n = n_blk + nl;
            const int64_t mm = (int64_t)mt * 8 + m;
            if (n < p.N && mm < p.M) {
                // split order, 8 partial sums in flight at a time (not a chain of dependent L2 round trips)
                const float *base = p.partial + mm * p.N + n;
                const size_t split_stride = (size_t)Mp * p.N;
                float s = 0.f;
                for (int sp0 = 0; sp0 < p.split_k; sp0 += 8) {
                    float v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = (sp0 + j < p.split_k) ? __ldcg(base + (size_t)(sp0 + j) * split_stride) : 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) s += v[j];
                }
                if constexpr (AR) s_tile[u] = s;
                else store_out(p.Y, p.out_dtype, mm * p.N + n, s);
            }
        }
        if (AR) __syncthreads();
    }

    if constexpr (AR) {
        // ar_epoch counts the calls completed on this comm (same value on every rank); it was read after the
        // dependency wait, i.e. after the previous call on this rank had finished and advanced it.
        if (tid == 0) s_ar_fail = 0;
        __syncthreads();
        // 1. push this block's elements to every rank, two neighbouring columns per 16-byte store
        for (int u = tid; u < (GEMV_ROWS_PER_BLOCK / 2) * m_rows; u += GEMV_THREADS) {
            const int nl = 2 * (u & (GEMV_ROWS_PER_BLOCK / 2 - 1));
            const int m = u / (GEMV_ROWS_PER_BLOCK / 2);
            const int64_t n = n_blk + nl;
            const int64_t mm = (int64_t)mt * 8 + m;
            if (n < p.N && mm < p.M)
                exch_push2(ar, ar_epoch, (size_t)(mm * p.N + n), s_tile[m * GEMV_ROWS_PER_BLOCK + nl],
                           s_tile[m * GEMV_ROWS_PER_BLOCK + nl + 1]);
        }
        // 2. collect every rank's pairs for the same elements and write the output
        if (!exch_collect_tile(ar, ar_epoch, (int64_t)mt * 8, m_rows, n_blk, GEMV_ROWS_PER_BLOCK, p.M, p.N, p.Y,
                               p.out_dtype, tid, GEMV_THREADS, &s_ar_fail))
            s_ar_fail = 1;
        __syncthreads();
        if (tid == 0) exch_block_done(ar, ar_epoch, gridDim.x * gridDim.z, s_ar_fail != 0);
    }
}

// Two entry points over one body: the plain kernel keeps its one-struct parameter block; the exchanging kernel
// adds the ArParams.
template <bool BF16, int ZMODE, int MPAD>
__global__ void __launch_bounds__(GEMV_THREADS, 4) gemv_kernel(const GemvParams p) {
    gemv_body<BF16, ZMODE, MPAD, false>(p, NoExchange{});
}
template <bool BF16, int ZMODE, int MPAD>
__global__ void __launch_bounds__(GEMV_THREADS, 4) gemv_exch_kernel(const GemvParams p, const ArParams ar) {
    gemv_body<BF16, ZMODE, MPAD, true>(p, ar);
}

template <bool BF16, int ZMODE, int MPAD>
static cudaError_t set_attr1() {
    const int bytes = (int)gemv_smem_bytes(GEMV_MAX_CHUNKS_PER_SPLIT, MPAD);
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<BF16, ZMODE, MPAD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemv_exch_kernel<BF16, ZMODE, MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 bytes);
    return e;
}
template <bool BF16, int ZMODE>
static cudaError_t set_attr() {
    cudaError_t e = set_attr1<BF16, ZMODE, 1>();
    if (e == cudaSuccess) e = set_attr1<BF16, ZMODE, 2>();
    if (e == cudaSuccess) e = set_attr1<BF16, ZMODE, 4>();
    if (e == cudaSuccess) e = set_attr1<BF16, ZMODE, 8>();
    return e;
}

int gemv_init(qf_ctx *ctx) {
    QF_CUDA_TRY(ctx, (set_attr<false, QF_ZERO_CONST>()));
    QF_CUDA_TRY(ctx, (set_attr<false, QF_ZERO_U4>()));
    QF_CUDA_TRY(ctx, (set_attr<false, QF_ZERO_I8>()));
    QF_CUDA_TRY(ctx, (set_attr<true, QF_ZERO_CONST>()));
    QF_CUDA_TRY(ctx, (set_attr<true, QF_ZERO_U4>()));
    QF_CUDA_TRY(ctx, (set_attr<true, QF_ZERO_I8>()));
    return QF_OK;
}

// Plain launch; p.cluster_reduce groups the split_k blocks of a column block into a thread-block cluster.
static cudaError_t gemv_launch_plain(void (*kernel)(GemvParams), dim3 grid, dim3 blk, size_t smem, cudaStream_t s,
                                     bool pdl, const GemvParams &p) {
    const dim3 cl(1, p.cluster_reduce ? (unsigned)p.split_k : 1u, 1);
    return launch_kernel_cluster(kernel, grid, blk, smem, s, pdl, cl, p);
}

template <bool BF16, int ZMODE>
static cudaError_t gemv_dispatch_m(dim3 grid, size_t smem, cudaStream_t s, const GemvParams &p, const ArParams *ar) {
    const dim3 blk(GEMV_THREADS);
    const bool pdl = pdl_enabled();
    if (ar) {
        switch (p.m_pad) {
            case 1: return launch_kernel(gemv_exch_kernel<BF16, ZMODE, 1>, grid, blk, smem, s, pdl, p, *ar);
            case 2: return launch_kernel(gemv_exch_kernel<BF16, ZMODE, 2>, grid, blk, smem, s, pdl, p, *ar);
            case 4: return launch_kernel(gemv_exch_kernel<BF16, ZMODE, 4>, grid, blk, smem, s, pdl, p, *ar);
            default: return launch_kernel(gemv_exch_kernel<BF16, ZMODE, 8>, grid, blk, smem, s, pdl, p, *ar);
        }
    }
    switch (p.m_pad) {
        case 1: return gemv_launch_plain(gemv_kernel<BF16, ZMODE, 1>, grid, blk, smem, s, pdl, p);
        case 2: return gemv_launch_plain(gemv_kernel<BF16, ZMODE, 2>, grid, blk, smem, s, pdl, p);
        case 4: return gemv_launch_plain(gemv_kernel<BF16, ZMODE, 4>, grid, blk, smem, s, pdl, p);
        default: return gemv_launch_plain(gemv_kernel<BF16, ZMODE, 8>, grid, blk, smem, s, pdl, p);
    }
}
template <bool BF16>
static cudaError_t gemv_dispatch(int zmode, dim3 grid, size_t smem, cudaStream_t s, const GemvParams &p,
                                 const ArParams *ar) {
    if (zmode == QF_ZERO_CONST) return gemv_dispatch_m<BF16, QF_ZERO_CONST>(grid, smem, s, p, ar);
    if (zmode == QF_ZERO_U4) return gemv_dispatch_m<BF16, QF_ZERO_U4>(grid, smem, s, p, ar);
    return gemv_dispatch_m<BF16, QF_ZERO_I8>(grid, smem, s, p, ar);
}

static int launch_gemv_impl(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                            const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s,
                            const ArParams *ar) {
    GemvParams p;
    p.X = (const uint16_t *)X;
    p.qw = (const uint32_t *)qw;
    p.scales = (const uint16_t *)scales;
    p.zeros = zeros;
    p.Y = Y;
    p.counters = (int *)ws;  // fixed-size counter region first, partial sums after it
    p.partial = (float *)((char *)ws + plan.ws_counter_bytes);
    p.M = d->M;
    p.N = d->N;
    p.K = d->K;
    p.group_chunks = d->group_size / 128;
    p.chunks = (int)(d->K / 128);
    p.chunks_per_split = plan.chunks_per_split;
    p.split_k = plan.split_k;
    p.out_dtype = d->out_dtype;
    p.zero_const = d->zero_const;
    // 2..8 short splits: one thread-block cluster per column block sums the partial outputs on chip. The blocks of a
    // cluster leave together, so with long splits the slots they hold cost more than the global-memory tail saves
    // (measured: M=1 4096x4096, 4 chunks per split, 6.9 -> 6.5 us; 4096x14336 and 14336x4096, 11-14 chunks, 3-4 % slower).
    // Clusters are placed inside one GPC, so a launch close to the 592 block slots would spill into a second wave.
    const int64_t blocks = (int64_t)((d->N + GEMV_ROWS_PER_BLOCK - 1) / GEMV_ROWS_PER_BLOCK) * plan.split_k * plan.m_tiles;
    p.cluster_reduce = (!ar && plan.split_k >= 2 && plan.split_k <= 8 && plan.chunks_per_split <= 8 &&
                        blocks <= 512 && cluster_reduce_enabled())
                           ? 1
                           : 0;
    dim3 grid((unsigned)((d->N + GEMV_ROWS_PER_BLOCK - 1) / GEMV_ROWS_PER_BLOCK), (unsigned)plan.split_k,
              (unsigned)plan.m_tiles);
    const int64_t m_in_tile = d->M < 8 ? d->M : 8;
    p.m_pad = m_in_tile <= 1 ? 1 : m_in_tile <= 2 ? 2 : m_in_tile <= 4 ? 4 : 8;
    const size_t smem = gemv_smem_bytes(plan.chunks_per_split, p.m_pad);
    const cudaError_t le = d->act_dtype == QF_BF16 ? gemv_dispatch<true>(d->zero_mode, grid, smem, s, p, ar)
                                                   : gemv_dispatch<false>(d->zero_mode, grid, smem, s, p, ar);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, le);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

int launch_gemv(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s) {
    return launch_gemv_impl(ctx, d, plan, X, qw, scales, zeros, Y, ws, s, nullptr);
}

int launch_gemv_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                   const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s, const ArParams &ar) {
    return launch_gemv_impl(ctx, d, plan, X, qw, scales, zeros, Y, ws, s, &ar);
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate: the split-K scratch is a static device array.
// ---------------------------------------------------------------------------------------------
// In host code the name below is only a handle for the symbol, not a device address; the address each
// device uses is looked up once per device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) unsigned char g_static_scratch[QF_STATIC_SCRATCH_BYTES];

static std::mutex g_static_mutex;
static void *g_static_ptr[64] = {nullptr};  // per device ordinal

// Device address of the static scratch on the CURRENT device; first use per device also raises the
// kernels' dynamic shared-memory limit. Neither step allocates.
static int static_scratch_for_current_device(qf_ctx *ctx, void **out) {
    int dev = -1;
    QF_CUDA_TRY(ctx, cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(ctx, QF_ERR_UNSUPPORTED, "device ordinal out of range");
    std::lock_guard<std::mutex> g(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *ptr = nullptr;
        QF_CUDA_TRY(ctx, cudaGetSymbolAddress(&ptr, g_static_scratch));
        int st = gemv_init(ctx);
        if (st != QF_OK) return st;
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return QF_OK;
}

int launch_gemv_static(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                       const void *scales, const void *zeros, void *Y, cudaStream_t s) {
    const size_t need = plan.ws_partial_bytes + plan.ws_counter_bytes;
    if (need > (size_t)QF_STATIC_SCRATCH_BYTES)
        return fail(ctx, QF_ERR_WORKSPACE,
                    "this linear needs " + std::to_string(need) + " bytes of split-K scratch but the static array holds " +
                        std::to_string((size_t)QF_STATIC_SCRATCH_BYTES) +
                        (d->K <= 128 * GEMV_MAX_CHUNKS_PER_SPLIT
                             ? "; request split_k = 1 (no scratch at all for this K) or use qf_w4a16_linear with a caller "
                               "workspace"
                             : "; use qf_w4a16_linear with a caller workspace (K this long is always split)"));
    void *scratch = nullptr;
    int st = static_scratch_for_current_device(ctx, &scratch);
    if (st != QF_OK) return st;
    if (need > 0) {
        // the array keeps the previous call's contents: the arrival counters this launch uses must start at zero
        const size_t n_counters = (size_t)((d->N + GEMV_ROWS_PER_BLOCK - 1) / GEMV_ROWS_PER_BLOCK) * plan.m_tiles;
        QF_CUDA_TRY(ctx, cudaMemsetAsync(scratch, 0, n_counters * sizeof(int), s));
    }
    return launch_gemv(ctx, d, plan, X, qw, scales, zeros, Y, scratch, s);
}

}  // namespace qf
