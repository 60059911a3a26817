// K2: W4A16 GEMV / skinny GEMM (batch tile of 8 rows of X), HBM-bound.
//
// Y[M,N] = X[M,K] . W^T with W dequantised in registers and never written to memory.
//
// Work split
//   grid.x : blocks of 64 output columns (4 warps x 16 weight rows)
//   grid.y : K splits (split-K); partial sums meet in caller-provided fp32 scratch, the last
//            block to arrive for a column block sums them in split order (deterministic)
//   grid.z : batch tiles of 8 rows of X
// Per warp and 128-code chunk of K: every lane loads 16 B (32 codes) of weight row g = lane/4
// and of row g+8 with 128-bit loads that bypass L1 (the 4 lanes of a row cover 64 contiguous
// bytes), converts them with lop3 / packed-half arithmetic (zero and scale applied in registers)
// into the A fragments of eight m16n8k16 tensor-core MMAs, whose B fragments are the activations.
// The contraction index may be permuted freely as long as A and B agree, so the code pairs come
// out of the converter as (c_i, c_{i+4}) and the activations are staged ONCE per block into
// shared memory in that same order; no per-weight shuffle is spent on ordering.
// Accumulation is fp32 in the MMA accumulators.
#include <mutex>

#include "qf_common.cuh"

namespace qf {

constexpr int GEMV_THREADS = 128;
constexpr int GEMV_WARPS = 4;
constexpr int GEMV_ROWS_PER_BLOCK = 16 * GEMV_WARPS;  // 64
constexpr int GEMV_CB = 4;                            // chunks (of 128 codes) per register batch
constexpr int GEMV_MAX_CHUNKS_PER_SPLIT = 48;         // 2 KB of staged activations per chunk

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
};

template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    if (BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// One register batch: weights of rows g / g+8 for up to GEMV_CB chunks plus their scales and zeros.
struct WBatch {
    uint4 wa[GEMV_CB], wb[GEMV_CB];
    uint32_t sc[GEMV_CB];  // scale(row g) | scale(row g+8) << 16
    int z[GEMV_CB];        // zero(row g) & 0xffff | zero(row g+8) << 16  (signed 16-bit fields)
};

template <int ZMODE>
__device__ __forceinline__ void load_batch(WBatch &b, const GemvParams &p, int64_t row_a, int c_begin, int c_end,
                                           int t) {
    const int64_t words_per_row = p.K >> 3;
    const uint32_t *ra = p.qw + row_a * words_per_row + t * 4;
    const uint32_t *rb = ra + 8 * words_per_row;
#pragma unroll
    for (int i = 0; i < GEMV_CB; ++i) {
        const int c = c_begin + i;
        if (c < c_end) {
            b.wa[i] = ldg_stream(ra + (int64_t)c * 16);
            b.wb[i] = ldg_stream(rb + (int64_t)c * 16);
        }
    }
#pragma unroll
    for (int i = 0; i < GEMV_CB; ++i) {
        const int c = c_begin + i;
        if (c < c_end) {
            const int64_t gi = c / p.group_chunks;
            const uint32_t sa = __ldg(p.scales + gi * p.N + row_a);
            const uint32_t sb = __ldg(p.scales + gi * p.N + row_a + 8);
            b.sc[i] = sa | (sb << 16);
            const int za = load_zero<ZMODE>(p.zeros, p.zero_const, gi, row_a, p.N);
            const int zb = load_zero<ZMODE>(p.zeros, p.zero_const, gi, row_a + 8, p.N);
            b.z[i] = (za & 0xffff) | (zb << 16);
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void compute_batch(const WBatch &b, float (&acc)[2][4], const uint4 *xs, int c_local_begin,
                                              int n_valid, int lane) {
#pragma unroll
    for (int i = 0; i < GEMV_CB; ++i) {
        if (i < n_valid) {
            ZeroScale<BF16> za, zb;
            za.set((int)(short)(b.z[i] & 0xffff), b.sc[i] & 0xffffu);
            zb.set(b.z[i] >> 16, b.sc[i] >> 16);
            const uint32_t wa[4] = {b.wa[i].x, b.wa[i].y, b.wa[i].z, b.wa[i].w};
            const uint32_t wb[4] = {b.wb[i].x, b.wb[i].y, b.wb[i].z, b.wb[i].w};
            const uint4 *xc = xs + (size_t)(c_local_begin + i) * 128 + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t pa[4], pb[4];
                dequant8<BF16>(wa[j], za, pa);
                dequant8<BF16>(wb[j], zb, pb);
                const uint4 xb = xc[j * 32];
                mma_16816<BF16>(acc[0], pa[0], pb[0], pa[1], pb[1], xb.x, xb.y);
                mma_16816<BF16>(acc[1], pa[2], pb[2], pa[3], pb[3], xb.z, xb.w);
            }
        }
    }
}

template <bool BF16, int ZMODE>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ uint4 xs[];  // [chunk_local][j][m 0..7][t 0..3]
    __shared__ int s_is_last;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int split = blockIdx.y;
    const int mt = blockIdx.z;
    const int c0 = split * p.chunks_per_split;
    const int c1 = min(c0 + p.chunks_per_split, p.chunks);
    const int64_t n_blk = (int64_t)blockIdx.x * GEMV_ROWS_PER_BLOCK;
    const int64_t row_a = n_blk + warp * 16 + g;
    const bool warp_active = (n_blk + warp * 16) < p.N;  // N is a multiple of 16

    // 1. first weight batch in flight before anything else
    WBatch A, B;
    if (warp_active) load_batch<ZMODE>(A, p, row_a, c0, c1, t);

    // 2. stage the activations of this K range in fragment order, zero rows beyond M
    {
        const int n_units = (c1 - c0) * 128;  // uint4 units: chunk x (m 8) x (16 B pieces 16)
        const int64_t m_base = (int64_t)mt * 8;
        for (int u = tid; u < n_units; u += GEMV_THREADS) {
            const int piece = u & 15;  // = t*4 + j : 16-byte piece of the chunk's 256-byte row segment
            const int m = (u >> 4) & 7;
            const int cl = u >> 7;
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
            xs[((cl * 4 + j) * 8 + m) * 4 + tt] = r;
        }
    }
    __syncthreads();

    // 3. main loop, register double buffering
    float acc2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // two chains: MMAs of one chain are dependent
    if (warp_active) {
        for (int c = c0; c < c1; c += 2 * GEMV_CB) {
            const bool has_b = (c + GEMV_CB) < c1;
            if (has_b) load_batch<ZMODE>(B, p, row_a, c + GEMV_CB, c1, t);
            compute_batch<BF16>(A, acc2, xs, c - c0, min(GEMV_CB, c1 - c), lane);
            if (has_b) {
                if (c + 2 * GEMV_CB < c1) load_batch<ZMODE>(A, p, row_a, c + 2 * GEMV_CB, c1, t);
                compute_batch<BF16>(B, acc2, xs, c + GEMV_CB - c0, min(GEMV_CB, c1 - c - GEMV_CB), lane);
            }
        }
    }

    // 4. epilogue. acc[0..1]: row g, batch 2t, 2t+1 ; acc[2..3]: row g+8
    float acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = acc2[0][i] + acc2[1][i];
    const int64_t m0 = (int64_t)mt * 8 + 2 * t;
    if (p.split_k == 1) {
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

    const int64_t Mp = (int64_t)gridDim.z * 8;
    if (warp_active) {
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
    for (int u = tid; u < GEMV_ROWS_PER_BLOCK * 8; u += GEMV_THREADS) {
        const int nl = u & (GEMV_ROWS_PER_BLOCK - 1);
        const int m = u / GEMV_ROWS_PER_BLOCK;
        const int64_t n = n_blk + nl;
        const int64_t mm = (int64_t)mt * 8 + m;
        if (n < p.N && mm < p.M) {
            float s = 0.f;
            for (int sp = 0; sp < p.split_k; ++sp) s += __ldcg(p.partial + ((int64_t)sp * Mp + mm) * p.N + n);
            store_out(p.Y, p.out_dtype, mm * p.N + n, s);
        }
    }
}

template <bool BF16, int ZMODE>
static cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemv_kernel<BF16, ZMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GEMV_MAX_CHUNKS_PER_SPLIT * 2048);
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

template <bool BF16>
static void gemv_dispatch(int zmode, dim3 grid, size_t smem, cudaStream_t s, const GemvParams &p) {
    if (zmode == QF_ZERO_CONST)
        gemv_kernel<BF16, QF_ZERO_CONST><<<grid, GEMV_THREADS, smem, s>>>(p);
    else if (zmode == QF_ZERO_U4)
        gemv_kernel<BF16, QF_ZERO_U4><<<grid, GEMV_THREADS, smem, s>>>(p);
    else
        gemv_kernel<BF16, QF_ZERO_I8><<<grid, GEMV_THREADS, smem, s>>>(p);
}

int launch_gemv(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s) {
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
    dim3 grid((unsigned)((d->N + GEMV_ROWS_PER_BLOCK - 1) / GEMV_ROWS_PER_BLOCK), (unsigned)plan.split_k,
              (unsigned)plan.m_tiles);
    const size_t smem = (size_t)plan.chunks_per_split * 2048;
    if (d->act_dtype == QF_BF16)
        gemv_dispatch<true>(d->zero_mode, grid, smem, s, p);
    else
        gemv_dispatch<false>(d->zero_mode, grid, smem, s, p);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
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
                        "; pass split_k = 1 or use qf_w4a16_linear with a caller workspace");
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
