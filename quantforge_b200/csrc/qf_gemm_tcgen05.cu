// K3: W4A16 GEMM on the 5th-generation tensor cores (tcgen05), weights dequantised in the mainloop.
//
// Computes Y^T = W . X^T tile by tile so that the DEQUANTISED WEIGHTS are the MMA's A operand and
// live only in tensor memory (TMEM):
//   MMA M = 128 output features (weight rows, one per TMEM lane)
//   MMA N = BN  rows of X (the batch), 16..256
//   MMA K = 16  per instruction, BK codes per pipeline stage
//
// Roles inside a CTA (320 threads):
//   warps 0-3, 4-7 : two converter groups, alternating k-blocks. Thread t of a group owns weight row
//                    n0 + t: it reads the row's packed codes from the TMA-staged shared-memory tile,
//                    converts them with lop3 / packed 16-bit arithmetic (zero and scale of its own
//                    row and group held in registers), and writes the 16-bit operand straight into
//                    TMEM lane t with tcgen05.st.  The same threads run the epilogue
//                    (tcgen05.ld -> convert -> global store, or split-K partials).
//   warp 8         : TMA producer (one elected thread): packed-weight tile and X tile per stage.
//   warp 9         : TMEM allocation and, one elected thread, tcgen05.mma issue: A from TMEM,
//                    B (= X tile, K-major, 128-byte swizzle) from shared memory, fp32 accumulate in TMEM.
// Every mbarrier wait is bounded: on expiry the CTA raises an abort flag, records QF_ERR_TIMEOUT in
// the context's status word, drains its own TMA copies, frees its TMEM and returns.
// Every CTA loads its own tiles (plain TMA loads). Split-K over 2..8 blocks runs as a thread-block cluster whose
// blocks sum their partial tiles through distributed shared memory; other splits use global partial tiles and an
// arrival counter. Both cluster barriers are passed by every block, aborted or not.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "qf_common.cuh"
#include "qf_mbar.cuh"

namespace qf {

// ---------------------------------------------------------------------------------------------
// configuration per batch-tile width
// ---------------------------------------------------------------------------------------------
template <int BN>
struct GemmCfg {
    static constexpr int BK = (BN <= 128) ? 128 : 64;           // codes per k-block
    static constexpr int W_ROW_BYTES = BK / 2;                   // 64 or 32
    static constexpr int W_STAGE_BYTES = 128 * W_ROW_BYTES;      // 8 KB or 4 KB
    static constexpr int X_BOX_BYTES = BN * 128;                 // one 64-element box
    static constexpr int X_STAGE_BYTES = X_BOX_BYTES * (BK / 64);
    static constexpr int STAGE_BYTES = W_STAGE_BYTES + X_STAGE_BYTES;
    static constexpr int STAGES = BN == 16 ? 8 : BN == 32 ? 6 : BN == 64 ? 4 : 5;
    static constexpr int NA = BN <= 64 ? 3 : 4;                  // A operand buffers in TMEM
    static constexpr int A_COLS = BK / 2;                        // 32-bit TMEM columns per A buffer
    static constexpr int TMEM_COLS = (BN + NA * A_COLS) <= 256 ? 256 : 512;
    static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int SZ_BYTES = 512;                          // per stage: 256 B scales + up to 128 B zeros
    static constexpr int SMEM_BYTES =
        STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + STAGES * SZ_BYTES;
};

constexpr int GEMM_THREADS = 320;

struct GemmParams {
    const uint16_t *scales;
    const void *zeros;
    void *Y;
    float *partial;
    int *counters;
    int *status;  // host-mapped status word
    int64_t M, N, K;
    int group_size;
    int zero_mode, zero_const;
    int out_dtype;
    int kblocks;           // K / BK
    int kblocks_per_split;
    int split_k;
    int interleaved;       // weight nibble order inside a word: 0 canonical, 1 pair-interleaved
    int tiled;             // 1: weights stored tile-major (QF_LAYOUT_TILED)
    int cluster_reduce;    // 1: the split_k blocks of a tile form a thread-block cluster and sum their partial
                           //    tiles through distributed shared memory (no global partials, no counters)
    const void *residual;  // QF_EPI_RESIDUAL_ADD: R[M, N] in out_dtype
    int epilogue;          // qf_epilogue (plain instantiations only)
};

__device__ __forceinline__ float gemm_load_out(const void *R, int out_dtype, int64_t idx) {
    if (out_dtype == QF_F32) return reinterpret_cast<const float *>(R)[idx];
    if (out_dtype == QF_F16) return __half2float(reinterpret_cast<const __half *>(R)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(R)[idx]);
}
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.f + expf(-gate)) * up; }
// Four finished outputs of batch row m, weight rows n..n+3 (n a multiple of 4), with the plain or residual epilogue.
__device__ __forceinline__ void gemm_store4(const GemmParams &p, int64_t m, int64_t n, float4 a) {
    const int64_t o = m * p.N + n;
    if (p.epilogue == QF_EPI_RESIDUAL_ADD) {
        a.x += gemm_load_out(p.residual, p.out_dtype, o);
        a.y += gemm_load_out(p.residual, p.out_dtype, o + 1);
        a.z += gemm_load_out(p.residual, p.out_dtype, o + 2);
        a.w += gemm_load_out(p.residual, p.out_dtype, o + 3);
    }
    store_out(p.Y, p.out_dtype, o, a.x);
    store_out(p.Y, p.out_dtype, o + 1, a.y);
    store_out(p.Y, p.out_dtype, o + 2, a.z);
    store_out(p.Y, p.out_dtype, o + 3, a.w);
}
// QF_EPI_SILU_MUL: weight rows n..n+3 (n % 16 < 8) are gate rows, n+8.. the matching up rows; output column
// (n / 16) * 8 + n % 8 of Y[M, N/2].
__device__ __forceinline__ void gemm_store4_silu(const GemmParams &p, int64_t m, int64_t n, float4 g, float4 u) {
    const int64_t o = m * (p.N >> 1) + (n >> 4) * 8 + (n & 7);
    store_out(p.Y, p.out_dtype, o, silu_mul(g.x, u.x));
    store_out(p.Y, p.out_dtype, o + 1, silu_mul(g.y, u.y));
    store_out(p.Y, p.out_dtype, o + 2, silu_mul(g.z, u.z));
    store_out(p.Y, p.out_dtype, o + 3, silu_mul(g.w, u.w));
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// D[tmem] (+)= A[tmem] . B[smem desc]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One lane of a fully active warp (the same lane every time within a kernel).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// Arrives on the mbarrier once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// K-major shared-memory operand descriptor, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);        // start address
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset
    d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ int load_zero_rt(const void *zeros, int zmode, int zconst, int64_t gi, int64_t n,
                                            int64_t N) {
    if (zmode == QF_ZERO_CONST) return zconst;
    if (zmode == QF_ZERO_U4) return load_zero<QF_ZERO_U4>(zeros, zconst, gi, n, N);
    return load_zero<QF_ZERO_I8>(zeros, zconst, gi, n, N);
}

// 4 packed words (32 codes along K) -> 16 registers of 16-bit pairs in natural k order.
template <bool BF16, bool INTER>
__device__ __forceinline__ void convert32(const uint4 &v, const ZeroScale<BF16> &zs, uint32_t (&out)[16]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t p[4];
        dequant8<BF16>(w[j], zs, p);  // p[i] = (nibble i, nibble i+4)
        if (INTER) {                  // nibble order c0 c2 c4 c6 c1 c3 c5 c7: pairs are already (c0,c1)(c2,c3)..
            out[4 * j + 0] = p[0];
            out[4 * j + 1] = p[1];
            out[4 * j + 2] = p[2];
            out[4 * j + 3] = p[3];
        } else {
            out[4 * j + 0] = prmt(p[0], p[1], 0x5410u);
            out[4 * j + 1] = prmt(p[2], p[3], 0x5410u);
            out[4 * j + 2] = prmt(p[0], p[1], 0x7632u);
            out[4 * j + 3] = prmt(p[2], p[3], 0x7632u);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------
// EXCH: finished tiles are exchanged across GPUs (sum or gather) before Y is written; `ar` then is an ArParams.
// The plain instantiations take an empty struct instead, so their parameter block and code stay what they were.
template <bool BF16, int BN, bool INTER, bool EXCH>
__global__ void __launch_bounds__(GEMM_THREADS, GemmCfg<BN>::CTAS_PER_SM)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
            const GemmParams p, const typename ExchArg<EXCH>::type ar) {
    using C = GemmCfg<BN>;
    constexpr int BK = C::BK;
    constexpr int STAGES = C::STAGES;
    constexpr int NA = C::NA;
    constexpr bool CLUSTER_OK = BN <= 64 && !EXCH;  // the cluster reduction serves the narrow split-K tiles

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_is_last;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto afull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto aempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + NA + a); };
    const uint32_t dfull_bar = bar_base + 8u * (2 * STAGES + 2 * NA);
    auto w_stage = [&](int s) { return smem_base + (uint32_t)s * C::STAGE_BYTES; };
    auto x_stage = [&](int s) { return smem_base + (uint32_t)s * C::STAGE_BYTES + C::W_STAGE_BYTES; };
    auto sz_stage = [&](int s) { return bar_base + 256u + (uint32_t)s * C::SZ_BYTES; };

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int m_tile = blockIdx.x;
    const int n_tile = blockIdx.y;
    const int split = blockIdx.z;
    const int kb0 = split * p.kblocks_per_split;
    const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks);
    const int nkb = kb1 - kb0;
    const int64_t n0 = (int64_t)n_tile * 128;
    const int64_t m0 = (int64_t)m_tile * BN;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 128 + 1);
        }
        for (int a = 0; a < NA; ++a) {
            mbar_init(afull_bar(a), 128);
            mbar_init(aempty_bar(a), 1);
        }
        mbar_init(dfull_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(&s_tmem_base), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    volatile int *abort_flag = &s_abort;
    griddep_launch_dependents();  // the next kernel may begin its own set-up and weight prefetch

    int producer_issued = 0;  // meaningful in the elected producer lane only
    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp runs the loop (uniform control flow); one elected lane issues the copies.
        const bool leader = elect_one();
        const uint32_t zbytes = p.zero_mode == QF_ZERO_U4 ? 64u : p.zero_mode == QF_ZERO_I8 ? 128u : 0u;
        const uint32_t tx_bytes = C::STAGE_BYTES + 256u + zbytes;
        const int group_kb = p.group_size / BK;  // k-blocks per quantisation group (>= 1)
        const int gi = kb0 / group_kb;
        const uint8_t *sc_ptr = (const uint8_t *)(p.scales + n0) + (size_t)gi * p.N * 2;
        const size_t z_row = p.zero_mode == QF_ZERO_U4 ? (size_t)p.N / 2 : (size_t)p.N;
        const uint8_t *z_ptr =
            (const uint8_t *)p.zeros + (p.zero_mode == QF_ZERO_U4 ? (size_t)n0 / 2 : (size_t)n0) + (size_t)gi * z_row;
        const int w_row0 = p.tiled ? n_tile * (int)(p.K >> 7) * 128 : (int)n0;
        // issue_w is called for it = 0, 1, 2, ... in order: the sliver pointers advance incrementally
        int g_rem = kb0 % group_kb;
        auto issue_w = [&](int it, int s) {
            const int kb = kb0 + it;
            const uint32_t fb = full_bar(s);
            mbar_arrive_expect_tx(fb, tx_bytes);
            if (p.tiled) {
                // tile-major weights: rows of 64 bytes, the 128 rows of (n_tile, 128-code block) adjacent
                const int kb128 = (kb * BK) >> 7;
                tma_load_2d(w_stage(s), &tmap_w, fb, (BK == 128) ? 0 : (kb & 1) * 32, w_row0 + kb128 * 128);
            } else {
                tma_load_2d(w_stage(s), &tmap_w, fb, kb * C::W_ROW_BYTES, w_row0);
            }
            bulk_load(sz_stage(s), sc_ptr, 256u, fb);
            if (zbytes) bulk_load(sz_stage(s) + 256u, z_ptr, zbytes, fb);
            if (++g_rem == group_kb) {
                g_rem = 0;
                sc_ptr += (size_t)p.N * 2;
                z_ptr += z_row;
            }
        };
        auto issue_x = [&](int it, int s) {
            const int kb = kb0 + it;
#pragma unroll
            for (int b = 0; b < BK / 64; ++b)
                tma_load_2d(x_stage(s) + b * C::X_BOX_BYTES, &tmap_x, full_bar(s), kb * BK + b * 64, (int)m0);
            producer_issued = it + 1;
        };
        // First pass over the ring: weights, scales and zeros do not depend on the previous kernel of the stream,
        // so they are requested before the dependency wait; the activations after it.
        const int npre = min(STAGES, nkb);
        if (leader)
            for (int it = 0; it < npre; ++it) issue_w(it, it);
        griddep_wait();
        if (leader)
            for (int it = 0; it < npre; ++it) issue_x(it, it);
        int s = npre % STAGES;
        uint32_t ph = npre == STAGES ? 1u : 0u;
        for (int it = npre; it < nkb; ++it) {
            const bool ok = mbar_wait(empty_bar(s), ph ^ 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) break;
            if (leader) {
                issue_w(it, s);
                issue_x(it, s);
            }
            if (++s == STAGES) {
                s = 0;
                ph ^= 1;
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        const bool leader = elect_one();
        const uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                               ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint64_t desc_hi = make_b_desc(0) & 0xFFFFFFFF00000000ull;
        const uint32_t desc_lo_const = (uint32_t)(make_b_desc(0) & 0xFFFFFFFFull);
        int s = 0, a = 0;
        uint32_t ph = 0, aph = 0;
        for (int it = 0; it < nkb; ++it) {
            bool ok = mbar_wait(full_bar(s), ph, abort_flag);
            ok = ok && mbar_wait(afull_bar(a), aph, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) break;
            tc_fence_after();
            if (leader) {
                const uint32_t a_tmem = tmem_base + BN + a * C::A_COLS;
                const uint32_t lo0 = desc_lo_const | ((x_stage(s) >> 4) & 0x3FFFu);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    const uint32_t lo = lo0 + (uint32_t)(((kk >> 2) * C::X_BOX_BYTES + (kk & 3) * 32) >> 4);
                    umma_ts(tmem_base, a_tmem + kk * 8, desc_hi | lo, idesc, (kk > 0) ? 1u : (it > 0 ? 1u : 0u));
                }
                umma_commit(empty_bar(s));
                umma_commit(aempty_bar(a));
                if (it == nkb - 1) umma_commit(dfull_bar);
            }
            if (++s == STAGES) {
                s = 0;
                ph ^= 1;
            }
            if (++a == NA) {
                a = 0;
                aph ^= 1;
            }
        }
    } else {
        // ------------------------------ converters ------------------------------
        const int wg = warp >> 2;              // 0 or 1
        const int row = tid & 127;             // TMEM lane and weight row inside the tile
        const int64_t n = n0 + row;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        // swizzled 16-byte chunk positions of this row inside a weight stage
        const uint32_t row_off = (uint32_t)row * C::W_ROW_BYTES;
        const uint32_t sw = (BK == 128) ? ((row >> 1) & 3) : ((row >> 2) & 1);

        for (int it = wg; it < nkb; it += 2) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            const int a = it % NA;
            const uint32_t aph = (it / NA) & 1;
            // warp-uniform outcome: the tcgen05.st below is warp-collective
            bool ready = mbar_wait(full_bar(s), ph, abort_flag);
            ready = ready && mbar_wait(aempty_bar(a), aph ^ 1, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            // zero and scale of (this row, this k-block's group) from the stage's slivers
            ZeroScale<BF16> zs;
            {
                const uint32_t szb = sz_stage(s);
                uint32_t sbits;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sbits) : "r"(szb + 2u * row));
                int z = p.zero_const;
                if (p.zero_mode == QF_ZERO_U4) {
                    uint32_t zw;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(szb + 256u + 4u * (row >> 3)));
                    z = (int)((zw >> (4 * (row & 7))) & 0xFu);
                } else if (p.zero_mode == QF_ZERO_I8) {
                    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(z) : "r"(szb + 256u + row));
                }
                zs.set(z, sbits);
            }
            const uint32_t wbase = w_stage(s) + row_off;
            const uint32_t a_col = BN + a * C::A_COLS;
#pragma unroll
            for (int c = 0; c < C::W_ROW_BYTES / 16; ++c) {
                const uint4 v = lds128(wbase + (((uint32_t)c ^ sw) << 4));
                uint32_t out[16];
                convert32<BF16, INTER>(v, zs, out);
                tmem_st16(lane_taddr + a_col + c * 16, out);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(afull_bar(a));
            fence_proxy_async_shared();  // this thread's reads of the stage, before the copy engine refills it
            mbar_arrive(empty_bar(s));
        }

        // ------------------------------ epilogue ------------------------------
        const bool ok = __all_sync(0xffffffffu, mbar_wait(dfull_bar, 0, abort_flag));
        tc_fence_after();
        if (ok) {
            // the activations this tile consumed were requested after the dependency wait, so the previous call on
            // this rank has finished and advanced the epoch
            unsigned ar_epoch = 0u;
            if constexpr (EXCH) ar_epoch = exch_read_epoch(ar);
            constexpr int COLS_PER_WG = BN / 2;
            const int64_t Mp = (int64_t)gridDim.x * BN;
#pragma unroll 1
            for (int c8 = 0; c8 < COLS_PER_WG / 8; ++c8) {
                const int col = wg * COLS_PER_WG + c8 * 8;
                uint32_t r[8];
                tmem_ld8(lane_taddr + col, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int64_t m = m0 + col + j;
                    const float v = __uint_as_float(r[j]);
                    if (p.split_k == 1) {
                        if constexpr (EXCH) {
                            if (m < p.M) exch_push(ar, ar_epoch, (size_t)(m * p.N + n), v);
                        } else if (p.epilogue == QF_EPI_SILU_MUL) {
                            // lanes 0-7 and 16-23 of a warp hold gate rows, the lanes 8 above them the up rows
                            const float up = __shfl_xor_sync(0xffffffffu, v, 8);
                            if (m < p.M && (row & 8) == 0)
                                store_out(p.Y, p.out_dtype, m * (p.N >> 1) + (n >> 4) * 8 + (n & 7), silu_mul(v, up));
                        } else if (m < p.M) {
                            const float res =
                                p.epilogue == QF_EPI_RESIDUAL_ADD ? gemm_load_out(p.residual, p.out_dtype, m * p.N + n) : 0.f;
                            store_out(p.Y, p.out_dtype, m * p.N + n, v + res);
                        }
                    } else if (CLUSTER_OK && p.cluster_reduce) {
                        // partial tile [batch row][weight row] fp32 in the (now idle) pipeline stages
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_base + (uint32_t)((col + j) * 128 + row) * 4u),
                                     "f"(v)
                                     : "memory");
                    } else {
                        __stcg(p.partial + ((int64_t)split * Mp + m) * p.N + n, v);
                    }
                }
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (CLUSTER_OK && p.cluster_reduce) {
        // Split-K inside a cluster: the split_k blocks of this tile are the blocks of one cluster (rank = split).
        // Every block, aborted or not, passes both cluster barriers, so no block can wait for one that left.
        if (s_abort && warp == 8 && producer_issued > 0) {
            int dummy = 0;
            volatile int *no_abort = &dummy;
            for (int it = max(0, producer_issued - STAGES); it < producer_issued; ++it)
                mbar_wait(full_bar(it % STAGES), (it / STAGES) & 1, no_abort);
        }
        if (s_abort && tid == 0) atomicExch(p.status, QF_ERR_TIMEOUT);
        cluster_sync_all();  // all partial tiles are in shared memory
        if (!s_abort) {
            // each block sums its share of the tile from all blocks in split order and writes the output
            const int units = 32 * BN;  // float4 units of the tile
            const int per = (units + p.split_k - 1) / p.split_k;
            const int u_end = min(units, (split + 1) * per);
            for (int u = split * per + tid; u < u_end; u += GEMM_THREADS) {
                const int nl = (u & 31) * 4;
                const int64_t m = m0 + (u >> 5);
                const bool silu = p.epilogue == QF_EPI_SILU_MUL;
                if (m < p.M && !(silu && (nl & 8))) {
                    const uint32_t a = smem_base + (uint32_t)((u >> 5) * 128 + nl) * 4u;
                    float4 v[8];
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp)
                        v[sp] = sp < p.split_k ? ld_dsmem_f4(dsmem_addr(a, (uint32_t)sp)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp) {
                        acc.x += v[sp].x;
                        acc.y += v[sp].y;
                        acc.z += v[sp].z;
                        acc.w += v[sp].w;
                    }
                    if (silu) {
                        // the matching up rows sit 8 rows further on
#pragma unroll
                        for (int sp = 0; sp < 8; ++sp)
                            v[sp] = sp < p.split_k ? ld_dsmem_f4(dsmem_addr(a + 32u, (uint32_t)sp))
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                        float4 up = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int sp = 0; sp < 8; ++sp) {
                            up.x += v[sp].x;
                            up.y += v[sp].y;
                            up.z += v[sp].z;
                            up.w += v[sp].w;
                        }
                        gemm_store4_silu(p, m, n0 + nl, acc, up);
                    } else {
                        gemm_store4(p, m, n0 + nl, acc);
                    }
                }
            }
        }
        cluster_sync_all();  // nobody leaves while its tile may still be read
    } else if (s_abort) {
        if (warp == 8 && producer_issued > 0) {
            // drain this CTA's own TMA copies before the shared memory goes away
            int dummy = 0;
            volatile int *no_abort = &dummy;
            for (int it = max(0, producer_issued - STAGES); it < producer_issued; ++it)
                mbar_wait(full_bar(it % STAGES), (it / STAGES) & 1, no_abort);
        }
        if (tid == 0) atomicExch(p.status, QF_ERR_TIMEOUT);
        __syncthreads();
    } else {
        bool final_cta = true;  // this CTA holds (or has pushed) the finished tile
        unsigned ar_epoch = 0u;
        if constexpr (EXCH) ar_epoch = exch_read_epoch(ar);
        if (p.split_k > 1) {
            // split-K: last CTA of this (m_tile, n_tile) sums the partial tiles in split order
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                int *cnt = p.counters + (int64_t)n_tile * gridDim.x + m_tile;
                const int prev = atomicAdd(cnt, 1);
                s_is_last = (prev == p.split_k - 1);
                if (s_is_last) *cnt = 0;
            }
            __syncthreads();
            final_cta = s_is_last != 0;
            if (final_cta) {
                __threadfence();
                // Each thread owns 4 consecutive output columns (one 16-byte load per split) and keeps 4 splits in
                // flight, so the reduction is not a chain of dependent L2 round trips.
                const int64_t Mp = (int64_t)gridDim.x * BN;
                const size_t split_stride = (size_t)Mp * p.N;
                for (int u = tid; u < 32 * BN; u += GEMM_THREADS) {
                    const int nl = (u & 31) * 4;
                    const int64_t m = m0 + (u >> 5);
                    const bool silu = !EXCH && p.epilogue == QF_EPI_SILU_MUL;
                    if (m < p.M && !(silu && (nl & 8))) {
                        // sum over the splits of 4 consecutive output columns starting `off` columns into the row
                        auto sum4 = [&](int off) {
                            const float *base = p.partial + (size_t)m * p.N + n0 + nl + off;
                            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                            for (int sp0 = 0; sp0 < p.split_k; sp0 += 4) {
                                float4 v[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    v[j] = (sp0 + j < p.split_k)
                                               ? __ldcg(reinterpret_cast<const float4 *>(base + (size_t)(sp0 + j) * split_stride))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    acc.x += v[j].x;
                                    acc.y += v[j].y;
                                    acc.z += v[j].z;
                                    acc.w += v[j].w;
                                }
                            }
                            return acc;
                        };
                        const float4 acc = sum4(0);
                        const int64_t o = m * p.N + n0 + nl;
                        if constexpr (EXCH) {
                            exch_push2(ar, ar_epoch, (size_t)o, acc.x, acc.y);
                            exch_push2(ar, ar_epoch, (size_t)o + 2, acc.z, acc.w);
                        } else if (silu) {
                            gemm_store4_silu(p, m, n0 + nl, acc, sum4(8));
                        } else {
                            gemm_store4(p, m, n0 + nl, acc);
                        }
                    }
                }
            }
        }
        if constexpr (EXCH) if (final_cta) {
            // Cross-GPU step: every element of the tile has been pushed to all ranks (above, or in the epilogue);
            // collect the other ranks' values for the same elements and write the output. The pairs carry their
            // own arrival token, so no block-level synchronisation separates the pushes from the collects.
            if (!exch_collect_tile(ar, ar_epoch, m0, BN, n0, 128, p.M, p.N, p.Y, p.out_dtype, tid, GEMM_THREADS,
                                   abort_flag))
                s_abort = 1;
            __syncthreads();
            if (tid == 0) exch_block_done(ar, ar_epoch, gridDim.x * gridDim.y, s_abort != 0);
        }
    }
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}


// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

static EncodeTiledFn get_encode() {
    std::call_once(g_encode_once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            g_encode = (EncodeTiledFn)fn;
    });
    return g_encode;
}

struct MapKey {
    const void *ptr;
    uint64_t d0, d1;
    uint32_t b0, b1;
    int kind;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && b0 == o.b0 && b1 == o.b1 && kind == o.kind;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = std::hash<const void *>()(k.ptr);
        h ^= std::hash<uint64_t>()(k.d0 * 1000003u + k.d1) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
        h ^= std::hash<uint64_t>()(((uint64_t)k.b0 << 32) | k.b1 | ((uint64_t)k.kind << 60)) + (h << 6) + (h >> 2);
        return h;
    }
};
static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// 2-D row-major tensor map. kind 0: bytes (packed weights), 1: 16-bit elements (activations).
static int get_tensor_map(qf_ctx *ctx, CUtensorMap *out, const void *ptr, int kind, uint64_t inner, uint64_t outer,
                          uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    MapKey key{ptr, inner, outer, box_inner, box_outer, kind * 8 + (int)swz};
    {
        std::lock_guard<std::mutex> g(g_map_mutex);
        auto itf = g_maps.find(key);
        if (itf != g_maps.end()) {
            *out = itf->second;
            return QF_OK;
        }
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(ctx, QF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const uint64_t esize = kind == 0 ? 1 : 2;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * esize};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                     const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, QF_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    std::lock_guard<std::mutex> g(g_map_mutex);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = *out;
    return QF_OK;
}

constexpr bool gemm_has_exchange(int bn) { return bn <= 64; }  // the cross-GPU exchange serves decode batches only

template <bool BF16, int BN>
static cudaError_t gemm_set_attr() {
    const int bytes = GemmCfg<BN>::SMEM_BYTES;
    const cudaFuncAttribute attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BF16, BN, false, false>, attr, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_kernel<BF16, BN, true, false>, attr, bytes);
    if constexpr (gemm_has_exchange(BN)) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_kernel<BF16, BN, false, true>, attr, bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_kernel<BF16, BN, true, true>, attr, bytes);
    }
    return e;
}

int gemm_init(qf_ctx *ctx) {
    QF_CUDA_TRY(ctx, (gemm_set_attr<false, 16>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<false, 32>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<false, 64>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<false, 128>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<false, 256>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<true, 16>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<true, 32>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<true, 64>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<true, 128>()));
    QF_CUDA_TRY(ctx, (gemm_set_attr<true, 256>()));
    if (!ctx->host_status) {
        QF_CUDA_TRY(ctx, cudaHostAlloc((void **)&ctx->host_status, sizeof(int), cudaHostAllocMapped));
        *ctx->host_status = 0;
        QF_CUDA_TRY(ctx, cudaHostGetDevicePointer((void **)&ctx->dev_status, ctx->host_status, 0));
    }
    return QF_OK;
}

template <bool BF16, int BN>
static int gemm_launch_bn(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                          GemmParams &p, cudaStream_t s, const ArParams *ar) {
    using C = GemmCfg<BN>;
    CUtensorMap tw, tx;
    const bool tiled = d->weight_layout == QF_LAYOUT_TILED;
    int st = get_tensor_map(ctx, &tw, qw, 0, tiled ? 64 : (uint64_t)d->K / 2,
                            tiled ? (uint64_t)d->N * (uint64_t)(d->K / 128) : (uint64_t)d->N, C::W_ROW_BYTES, 128,
                            C::BK == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    if (st != QF_OK) return st;
    st = get_tensor_map(ctx, &tx, X, 1, (uint64_t)d->K, (uint64_t)d->M, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != QF_OK) return st;
    p.kblocks = (int)(d->K / C::BK);
    p.kblocks_per_split = plan.chunks_per_split;
    dim3 grid((unsigned)plan.m_tiles, (unsigned)(d->N / 128), (unsigned)plan.split_k);
    const dim3 blk(GEMM_THREADS);
    cudaError_t le;
    if (ar) {
        if constexpr (gemm_has_exchange(BN)) {
            le = p.interleaved ? launch_kernel(gemm_kernel<BF16, BN, true, true>, grid, blk, C::SMEM_BYTES, s,
                                               pdl_enabled(), tw, tx, p, *ar)
                               : launch_kernel(gemm_kernel<BF16, BN, false, true>, grid, blk, C::SMEM_BYTES, s,
                                               pdl_enabled(), tw, tx, p, *ar);
        } else {
            return fail(ctx, QF_ERR_UNSUPPORTED, "the in-kernel exchange serves M <= 64");
        }
    } else {
        // 2..8 splits of a narrow tile: one thread-block cluster per tile sums the partial tiles on chip
        // Clusters are placed inside one GPC, which leaves block slots unused where the GPC's slot count is not a
        // multiple of the cluster size; a launch that no longer fits in one wave loses more than the on-chip
        // reduction gains (measured: 32 x 8, 80 x 3, 112 x 2 blocks fit; 48 x 6 = 288 of the 296 slots do not).
        unsigned cluster_z = 1;
        if (BN <= 64 && plan.split_k >= 2 && plan.split_k <= 8 && cluster_reduce_enabled()) {
            if ((int64_t)grid.x * grid.y * grid.z <= kClusterMaxBlocks) {
                p.cluster_reduce = 1;
                cluster_z = (unsigned)plan.split_k;
            }
        }
        le = p.interleaved ? launch_kernel_cluster(gemm_kernel<BF16, BN, true, false>, grid, blk, C::SMEM_BYTES, s,
                                             pdl_enabled(), dim3(1, 1, cluster_z), tw, tx, p, NoExchange{})
                           : launch_kernel_cluster(gemm_kernel<BF16, BN, false, false>, grid, blk, C::SMEM_BYTES, s,
                                             pdl_enabled(), dim3(1, 1, cluster_z), tw, tx, p, NoExchange{});
    }
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, le);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

template <bool BF16>
static int gemm_launch_dt(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                          GemmParams &p, cudaStream_t s, const ArParams *ar) {
    switch (plan.bn) {
        case 16: return gemm_launch_bn<BF16, 16>(ctx, d, plan, X, qw, p, s, ar);
        case 32: return gemm_launch_bn<BF16, 32>(ctx, d, plan, X, qw, p, s, ar);
        case 64: return gemm_launch_bn<BF16, 64>(ctx, d, plan, X, qw, p, s, ar);
        case 128: return gemm_launch_bn<BF16, 128>(ctx, d, plan, X, qw, p, s, ar);
        case 256: return gemm_launch_bn<BF16, 256>(ctx, d, plan, X, qw, p, s, ar);
        default: return fail(ctx, QF_ERR_BAD_ARG, "bad batch tile");
    }
}

int gemm_block_k(int bn) { return bn <= 128 ? 128 : 64; }

static int launch_gemm_impl(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                            const void *scales, const void *zeros, void *Y, const void *residual, void *ws,
                            cudaStream_t s, const ArParams *ar) {
    GemmParams p;
    p.residual = residual;
    p.epilogue = ar ? QF_EPI_NONE : d->epilogue;
    p.scales = (const uint16_t *)scales;
    p.zeros = zeros;
    p.Y = Y;
    p.counters = (int *)ws;
    p.partial = (float *)((char *)ws + plan.ws_counter_bytes);
    p.status = ctx->dev_status;
    p.M = d->M;
    p.N = d->N;
    p.K = d->K;
    p.group_size = d->group_size;
    p.zero_mode = d->zero_mode;
    p.zero_const = d->zero_const;
    p.out_dtype = d->out_dtype;
    p.split_k = plan.split_k;
    p.interleaved = d->weight_layout != QF_LAYOUT_CANONICAL;
    p.tiled = d->weight_layout == QF_LAYOUT_TILED;
    p.cluster_reduce = 0;
    if (d->act_dtype == QF_BF16) return gemm_launch_dt<true>(ctx, d, plan, X, qw, p, s, ar);
    return gemm_launch_dt<false>(ctx, d, plan, X, qw, p, s, ar);
}

int launch_gemm(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                const void *scales, const void *zeros, void *Y, const void *residual, void *ws, cudaStream_t s) {
    return launch_gemm_impl(ctx, d, plan, X, qw, scales, zeros, Y, residual, ws, s, nullptr);
}

int launch_gemm_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *qw,
                   const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s, const ArParams &ar) {
    return launch_gemm_impl(ctx, d, plan, X, qw, scales, zeros, Y, nullptr, ws, s, &ar);
}

}  // namespace qf
