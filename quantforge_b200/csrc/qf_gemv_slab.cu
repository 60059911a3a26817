// K2s: streaming W4A16 GEMV / skinny GEMM (M <= 32) on QF_LAYOUT_GEMV_SLAB weights, HBM-bound.
//
// Y[M,N] = X[M,K] . W^T with W dequantised in registers (same converter as every other kernel here) and never
// written to memory.
//
// Work split. The weight matrix is cut into units of 64 rows x 128 codes (one QF_SLAB_UNIT_BYTES record of the
// blob: codes, scales and zeros of the unit, in consumption order). Units are numbered row block major, K chunk
// minor, and thread block i of G owns the CONTIGUOUS range [i*U/G, (i+1)*U/G): every block streams the same number
// of bytes (+-1 unit) from one contiguous range of HBM, whatever N and K are. G is a small multiple of the SM
// count, so the whole launch is resident at once.
//
// Inside a block (160 threads):
//   warp 4      producer: one cp.async.bulk per PAIR of consecutive units (8704 contiguous bytes of the blob) into a
//               ring of shared-memory stages (full / empty mbarriers), plus one 512-byte bulk copy per batch row for
//               the pair's slices of X (two of 256 bytes where the pair straddles a row block). All weight copies of
//               the first pass over the ring are issued BEFORE the programmatic-dependent-launch wait (weights do
//               not depend on the previous kernel of the stream), the activation copies after it.
//   warps 0-3   consumers: warp w owns rows 16w..16w+15 of the unit. Per unit and lane: 2 x 16 B of codes and two
//               constants words from shared memory -> lop3 / packed 16-bit arithmetic -> A fragments of
//               m16n8k16 tensor-core MMAs; B fragments are 16-byte reads of the natural-order activation slice
//               (the blob's nibble order makes adjacent codes adjacent halves of a register). fp32 accumulators.
//
// Row blocks whose K range is shared by several thread blocks (the ranges do not end on row-block boundaries):
// the thread block that holds the END of the row block's K range is its owner. It meets that segment first (its
// range starts in the middle of the row block), keeps the partial sums in registers and finishes the row block
// at the very end of its life; every other contributor leaves its partial sums in the workspace as 8-byte
// (value, token) words - no fence, no atomic, no wait on the contributor's side. The owner reads them (polling
// the tokens, bounded), sums in thread-block order (deterministic), writes Y and clears the tokens, which is what
// leaves the workspace ready for the next launch. An owner only ever waits for thread blocks with a LOWER index,
// which were dispatched before it.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "qf_common.cuh"
#include "qf_mbar.cuh"

namespace qf {

constexpr int SLAB_THREADS = 160;
constexpr int SLAB_TILE_BYTES = 1088;           // 2 x 512 B of codes + 64 B of constants
constexpr int SLAB_UNIT_BYTES = QF_SLAB_UNIT_BYTES;
constexpr int SLAB_X_PITCH = 576;               // bytes between batch rows of a stage's activation slices (2 x 256 + 64
                                                // of skew: rows g and g+1 land in different shared-memory banks)
constexpr int SLAB_MAX_DEPTH = 16;
static_assert(SLAB_UNIT_BYTES == 4 * SLAB_TILE_BYTES, "unit = 4 tiles");

struct SlabParams {
    const uint8_t *blob;
    const uint16_t *X;
    void *Y;
    const void *residual;
    unsigned long long *pairs;  // workspace: [G][4 warps][MT][32 lanes][4] (value | token << 32), zero between launches
    int *status;                // host-mapped status word of the context
    int64_t M, N, K;
    long long units;            // (N / 64) * (K / 128)
    int chunks;                 // K / 128
    int depth;                  // stages of the ring
    int m_pad;                  // batch rows a stage has room for: 1, 2, 4, 8, 16 or 32
    int out_dtype;
    int epilogue;
    int stream_only;            // measurement aid: consumers release every stage unread (see launch_gemv_slab_impl)
};

// Shared-memory loads with the constant part of the address as an immediate (no address arithmetic in the loop).
template <int OFF>
__device__ __forceinline__ uint32_t lds32_at(uint32_t base) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t base) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(base), "n"(OFF));
    return v;
}
// Two (value, token) words with one 16-byte access; each 8-byte word is written and read whole.
__device__ __forceinline__ void st_pairs2(unsigned long long *ptr, unsigned long long a, unsigned long long b) {
    asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(ptr), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_pairs2(const unsigned long long *ptr, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(ptr) : "memory");
}
__device__ __forceinline__ unsigned long long pair_of(float v) {
    return (unsigned long long)__float_as_uint(v) | (1ull << 32);
}

__device__ __forceinline__ float load_out(const void *R, int out_dtype, int64_t idx) {
    if (out_dtype == QF_F32) return reinterpret_cast<const float *>(R)[idx];
    if (out_dtype == QF_F16) return __half2float(reinterpret_cast<const __half *>(R)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(R)[idx]);
}

// Thread block that owns unit u under the partition [i*U/G, (i+1)*U/G): the largest i with i*U/G <= u.
__device__ __forceinline__ long long slab_cta_of(long long u, long long U, long long G) {
    return ((u + 1) * G - 1) / U;
}

template <bool BF16>
__device__ __forceinline__ ZeroScale<BF16> slab_consts(uint32_t word) {
    ZeroScale<BF16> zs;
    // low half / high half broadcast, written as register pack / unpack so that the assembler may fold the
    // broadcast into the operand selectors of the packed-half instructions that consume it
    asm("{.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tmov.b32 %0, {lo, lo};\n\tmov.b32 %1, {hi, hi};}"
        : "=r"(zs.zsub), "=r"(zs.s2)
        : "r"(word));
    // f16 only: -(64 + z) = (1024 + z) * (-1) + 960, exact in f16
    zs.zfma = BF16 ? 0u : fma_f16x2(zs.zsub, 0xbc00bc00u, 0x63806380u);
    return zs;
}

// Writes the finished 16 x M outputs a warp holds for weight rows n0 + {g, g+8} (lane = 4g + t owns batch rows
// nt*8 + 2t + {0, 1}).
template <int MT>
__device__ __forceinline__ void slab_store(const SlabParams &p, int64_t n0, int g, int t, const float (&v)[MT][4]) {
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t m = nt * 8 + 2 * t + e;
            if (m >= p.M) continue;
            if (p.epilogue == QF_EPI_SILU_MUL) {
                // rows g of the tile are gate rows, rows g+8 the matching up rows
                const float gate = v[nt][e], up = v[nt][2 + e];
                store_out(p.Y, p.out_dtype, m * (p.N >> 1) + (n0 >> 1) + g, gate / (1.f + expf(-gate)) * up);
            } else {
                const int64_t ia = m * p.N + n0 + g, ib = ia + 8;
                float a = v[nt][e], b = v[nt][2 + e];
                if (p.epilogue == QF_EPI_RESIDUAL_ADD) {
                    a += load_out(p.residual, p.out_dtype, ia);
                    b += load_out(p.residual, p.out_dtype, ib);
                }
                store_out(p.Y, p.out_dtype, ia, a);
                store_out(p.Y, p.out_dtype, ib, b);
            }
        }
}

// The cross-GPU step of the exchanging instantiations (row-parallel sum / column-parallel gather over NVLink peer
// memory, qf_w4a16_linear_allreduce / _allgather). A warp pushes every tile it finishes to all ranks at once, as
// (value, token) words, while its thread block keeps streaming; at the very end of the block's life it collects the
// other ranks' words for the tiles it finished - by then they have usually arrived - and writes Y.
template <int MT>
__device__ __forceinline__ void slab_push(const SlabParams &p, const ArParams &ar, unsigned epoch, int64_t n0, int g,
                                          int t, const float (&v)[MT][4]) {
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t m = nt * 8 + 2 * t + e;
            if (m < p.M) {
                exch_push(ar, epoch, (size_t)(m * p.N + n0 + g), v[nt][e]);
                exch_push(ar, epoch, (size_t)(m * p.N + n0 + g + 8), v[nt][2 + e]);
            }
        }
}
// Collects the 16 x M tile at weight rows n0.. from every rank's slot and writes it (sum in rank order, or each
// rank's values into its own column range). All 32 lanes call it; returns false when a wait ran out.
template <int MT>
__device__ __forceinline__ bool slab_collect(const SlabParams &p, const ArParams &ar, unsigned epoch, int64_t n0,
                                             int g, int t, volatile int *abort_flag) {
    const unsigned token = epoch + 1u;
    const uint2 *base = ar.local_slots + exch_parity_offset(ar, epoch);
    const long long t0 = clock64();
#pragma unroll 1
    for (int q = 0; q < MT * 2; ++q) {
        const int64_t m = (q >> 1) * 8 + 2 * t + (q & 1);
        const bool valid = m < p.M;
        const size_t ea = (size_t)(m * p.N + n0 + g), eb = ea + 8;
        uint2 va[kMaxPeers], vb[kMaxPeers];
        while (true) {
            bool miss = false;
            if (valid) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < ar.world) {
                        va[r] = ld_pair_sys(base + (size_t)r * ar.slot_elems + ea);
                        vb[r] = ld_pair_sys(base + (size_t)r * ar.slot_elems + eb);
                    }
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < ar.world && (va[r].y != token || vb[r].y != token)) miss = true;
            }
            if (!__any_sync(0xffffffffu, miss)) break;
            __nanosleep(100);
            if (__any_sync(0xffffffffu, clock64() - t0 > ar.wait_cycles || *abort_flag != 0)) return false;
        }
        if (!valid) continue;
        if (ar.gather) {
            const int64_t row = m * (p.N * ar.world) + n0 + g;
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < ar.world) {
                    store_out(p.Y, p.out_dtype, row + (int64_t)r * p.N, __uint_as_float(va[r].x));
                    store_out(p.Y, p.out_dtype, row + (int64_t)r * p.N + 8, __uint_as_float(vb[r].x));
                }
        } else {
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < ar.world) {
                    sa += __uint_as_float(va[r].x);
                    sb += __uint_as_float(vb[r].x);
                }
            store_out(p.Y, p.out_dtype, m * p.N + n0 + g, sa);
            store_out(p.Y, p.out_dtype, m * p.N + n0 + g + 8, sb);
        }
    }
    return true;
}

template <bool BF16, int MT, bool EXCH>
__device__ __forceinline__ void gemv_slab_body(const SlabParams &p, const typename ExchArg<EXCH>::type &ar) {
    extern __shared__ __align__(128) uint8_t slab_smem[];
    __shared__ int s_abort;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t stage_bytes = 2u * SLAB_UNIT_BYTES + (uint32_t)p.m_pad * SLAB_X_PITCH;
    const uint32_t ring = (smem_u32(slab_smem) + 127u) & ~127u;
    const uint32_t bar_base = ring + (uint32_t)p.depth * stage_bytes;
    auto stage = [&](int s) { return ring + (uint32_t)s * stage_bytes; };
    auto full_bar = [&](int s) { return bar_base + 16u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar_base + 16u * (uint32_t)s + 8u; };

    const long long G = gridDim.x;
    const long long cta = blockIdx.x;
    const long long u0 = cta * p.units / G;
    const int n_units = (int)((cta + 1) * p.units / G - u0);
    const int n_pairs = (n_units + 1) >> 1;
    volatile int *abort_flag = &s_abort;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < p.depth; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    griddep_launch_dependents();  // the next kernel of the stream may start its own weight prefetch

    if (warp == 4) {
        // ------------------------------ producer ------------------------------
        // A stage holds a PAIR of consecutive units (contiguous in the blob: one bulk copy) and their activation
        // slices; the last pair of an odd range holds one unit.
        const int M = (int)p.M;
        const uint8_t *src = p.blob + (size_t)u0 * SLAB_UNIT_BYTES;
        const int npre = min(p.depth, n_pairs);
        int issued = 0;
        auto pair_units = [&](int ip) { return min(2, n_units - 2 * ip); };
        auto issue_w = [&](int ip, int s) {  // lane 0
            const uint32_t nu = (uint32_t)pair_units(ip);
            mbar_arrive_expect_tx(full_bar(s), nu * ((uint32_t)SLAB_UNIT_BYTES + (uint32_t)M * 256u));
            bulk_load(stage(s), src + (size_t)ip * (2 * SLAB_UNIT_BYTES), nu * (uint32_t)SLAB_UNIT_BYTES, full_bar(s));
        };
        auto issue_x = [&](int ip, int s, int c) {  // lanes < M; c = K chunk of the pair's first unit
            const uint32_t dst = stage(s) + 2u * SLAB_UNIT_BYTES + (uint32_t)lane * SLAB_X_PITCH;
            const uint16_t *row = p.X + (size_t)lane * p.K;
            const int nu = pair_units(ip);
            if (nu == 2 && c + 1 < p.chunks) {
                bulk_load(dst, row + (size_t)c * 128, 512u, full_bar(s));
            } else {
                bulk_load(dst, row + (size_t)c * 128, 256u, full_bar(s));
                if (nu == 2) bulk_load(dst + 256u, row, 256u, full_bar(s));  // first chunk of the next row block
            }
        };
        if (lane == 0)
            for (int ip = 0; ip < npre; ++ip) issue_w(ip, ip);
        __syncwarp();
        griddep_wait();  // the activations are the previous kernel's output
        int c = (int)(u0 % p.chunks);
        auto advance_c = [&]() {
            c += 2;
            while (c >= p.chunks) c -= p.chunks;
        };
        for (int ip = 0; ip < npre; ++ip) {
            if (lane < M) issue_x(ip, ip, c);
            advance_c();
        }
        issued = npre;
        // steady state: ring position advances incrementally (npre == depth whenever this loop runs)
        int s = 0;
        uint32_t ph = 0;  // parity of the consumers' previous pass over stage s
        for (int ip = npre; ip < n_pairs; ++ip) {
            bool ok = mbar_try_wait(empty_bar(s), ph) != 0;
            if (!ok) ok = mbar_wait(empty_bar(s), ph, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) break;
            if (lane == 0) issue_w(ip, s);
            __syncwarp();
            if (lane < M) issue_x(ip, s, c);
            advance_c();
            issued = ip + 1;
            if (++s == p.depth) {
                s = 0;
                ph ^= 1u;
            }
        }
        if (s_abort) {
            // drain this block's own copies before its shared memory goes away (the consumers stopped waiting)
            int dummy = 0;
            volatile int *no_abort = &dummy;
            for (int ip = max(0, issued - p.depth); ip < issued; ++ip)
                mbar_wait(full_bar(ip % p.depth), (uint32_t)(ip / p.depth) & 1u, no_abort);
            if (lane == 0) atomicExch(p.status, QF_ERR_TIMEOUT);
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    griddep_wait();  // nothing to compute before the activations exist; the bounded waits below start after it
    // calls completed on this comm (same value on every rank): read after the previous call on this rank finished
    unsigned ar_epoch = 0u;
    if constexpr (EXCH) ar_epoch = exch_read_epoch(ar);
    long long first_done = -1, last_done = -1;  // row blocks this warp finished during the stream (a contiguous run)
    const int g = lane >> 2;
    const int t = lane & 3;
    float acc[MT][2][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][h][e] = 0.f;
    float held[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) held[nt][e] = 0.f;
    bool have_held = false;
    long long held_b = 0;
    long long b = u0 / p.chunks;
    int c = (int)(u0 % p.chunks);
    int c_lo = c;
    unsigned long long *my_pairs = p.pairs + (((size_t)cta * 4 + warp) * MT) * 128 + lane * 4;
    bool aborted = false;

    // Ring position and addresses advance incrementally (no division by the run-time depth in the loop).
    int s = 0;
    uint32_t ph = 0;
    uint32_t fbar = full_bar(0);
    uint32_t wptr = stage(0) + (uint32_t)warp * SLAB_TILE_BYTES + (uint32_t)lane * 16u;  // this lane's codes
    const uint32_t cst_off = 1024u + (uint32_t)g * 4u - (uint32_t)lane * 16u;            // -> its row's constants
    uint32_t x_off[MT];                                                                  // -> its activation rows
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        // batch rows beyond m_pad are never stored: wrap into the rows the stage holds
        const uint32_t row = (uint32_t)((nt * 8 + g) & (p.m_pad - 1));
        x_off[nt] = 2u * SLAB_UNIT_BYTES - (uint32_t)warp * SLAB_TILE_BYTES - (uint32_t)lane * 16u +
                    (uint32_t)t * 16u + row * SLAB_X_PITCH;
    }
    const uint32_t ring_bytes = (uint32_t)p.depth * stage_bytes;
    const uint32_t bars_bytes = 16u * (uint32_t)p.depth;
    int seg_left = min(p.chunks - c, n_units);

    if (p.stream_only) {
        // measurement aid: the bandwidth ceiling of the copy pipeline alone. Every stage is released unread; nothing is
        // converted, multiplied or written.
        for (int ip = 0; ip < n_pairs; ++ip) {
            if (!mbar_wait(fbar, ph, abort_flag)) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(fbar + 8u);
            fbar += 16u;
            if (++s == p.depth) {
                s = 0;
                ph ^= 1u;
                fbar = full_bar(0);
            }
        }
        return;
    }

    int units_left = n_units;
    int seg_len = seg_left;                                   // units of the current row-block segment
    const int odd_tail = (n_units & 1) ? n_pairs - 1 : -1;   // the pair that holds a single unit
    // one unit of the stage at wptr: UB = 0 for the first unit of the pair, 1 for the second (constant offsets)
    auto unit = [&](auto ub) {
        constexpr int WO = decltype(ub)::value * SLAB_UNIT_BYTES;
        constexpr int XO = decltype(ub)::value * 256;
        const uint4 va = lds128_at<WO>(wptr);
        const uint4 vb = lds128_at<WO + 512>(wptr);
        const uint32_t cptr = wptr + cst_off;
        const ZeroScale<BF16> za = slab_consts<BF16>(lds32_at<WO>(cptr));
        const ZeroScale<BF16> zb = slab_consts<BF16>(lds32_at<WO + 32>(cptr));
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
        const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t xptr[MT];
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) xptr[nt] = wptr + x_off[nt];
        auto step = [&](auto jc) {
            constexpr int j = decltype(jc)::value;
            uint32_t pa[4], pb[4];
            dequant8<BF16>(wa[j], za, pa);
            dequant8<BF16>(wb[j], zb, pb);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                const uint4 xb = lds128_at<XO + j * 64>(xptr[nt]);
                mma_16816<BF16>(acc[nt][0], pa[0], pb[0], pa[1], pb[1], xb.x, xb.y);
                mma_16816<BF16>(acc[nt][1], pa[2], pb[2], pa[3], pb[3], xb.z, xb.w);
            }
        };
        step(std::integral_constant<int, 0>{});
        step(std::integral_constant<int, 1>{});
        step(std::integral_constant<int, 2>{});
        step(std::integral_constant<int, 3>{});
    };
    // end of this block's share of a row block (or of its range)
    auto end_segment = [&]() {
            c += seg_len;
            units_left -= seg_len;
            // end of this block's share of row block b
            float v[MT][4];
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[nt][e] = acc[nt][0][e] + acc[nt][1][e];
                    acc[nt][0][e] = 0.f;
                    acc[nt][1][e] = 0.f;
                }
            if (c_lo == 0 && c == p.chunks) {
                if constexpr (EXCH) {
                    slab_push<MT>(p, ar, ar_epoch, b * 64 + warp * 16, g, t, v);
                    if (first_done < 0) first_done = b;
                    last_done = b;
                } else {
                    slab_store<MT>(p, b * 64 + warp * 16, g, t, v);
                }
            } else if (c == p.chunks) {
                // this block owns row block b (it holds the end of its K range): finished at the very end
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) held[nt][e] = v[nt][e];
                have_held = true;
                held_b = b;
            } else {
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    st_pairs2(my_pairs + nt * 128, pair_of(v[nt][0]), pair_of(v[nt][1]));
                    st_pairs2(my_pairs + nt * 128 + 2, pair_of(v[nt][2]), pair_of(v[nt][3]));
                }
            }
            if (c == p.chunks) {
                c = 0;
                ++b;
            }
            c_lo = c;
            seg_len = min(p.chunks - c, units_left);
            seg_left = seg_len;
    };

#pragma unroll 1
    for (int ip = 0; ip < n_pairs; ++ip) {
        if (!__all_sync(0xffffffffu, mbar_try_wait(fbar, ph) != 0)) {
            // not there yet for some lane: everybody takes the bounded wait
            if (!__all_sync(0xffffffffu, mbar_wait(fbar, ph, abort_flag))) {
                aborted = true;
                break;
            }
        }
        unit(std::integral_constant<int, 0>{});
        if (--seg_left == 0) end_segment();
        if (ip != odd_tail) {
            unit(std::integral_constant<int, 1>{});
            if (--seg_left == 0) end_segment();
        }
        // The stage is refilled by the copy engine (async proxy) once the four warps have released it, and the
        // reads above went through the generic proxy: the proxy fence orders them before the release. Without it the
        // last activation read of a step was observed to return the refill's data (thread blocks that start while
        // the memory system is lightly loaded, where a refill lands within a few hundred nanoseconds).
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive_at<8>(fbar);  // the stage's empty barrier sits right behind its full barrier
        wptr += stage_bytes;
        fbar += 16u;
        if (++s == p.depth) {
            s = 0;
            ph ^= 1u;
            wptr -= ring_bytes;
            fbar -= bars_bytes;
        }
    }

    if (aborted && lane == 0) atomicExch(p.status, QF_ERR_TIMEOUT);
    if (have_held && !aborted) {
        // contributors of row block held_b: the thread blocks from the one that holds its first unit up to cta - 1,
        // added in that order onto this block's own partial sums
        const long long first = slab_cta_of(held_b * p.chunks, p.units, G);
        constexpr int BATCH = MT == 1 ? 4 : MT == 2 ? 2 : 1;  // contributors whose words are in flight together
        const long long t0 = clock64();
        bool failed = false;
#pragma unroll 1
        for (long long j0 = first; j0 < cta; j0 += BATCH) {
            unsigned long long w[BATCH][MT][4];
            bool need[BATCH];
#pragma unroll
            for (int q = 0; q < BATCH; ++q) need[q] = j0 + q < cta;
            while (true) {
                bool miss = false;
#pragma unroll
                for (int q = 0; q < BATCH; ++q)
                    if (need[q]) {
                        const unsigned long long *src = p.pairs + (((size_t)(j0 + q) * 4 + warp) * MT) * 128 + lane * 4;
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) {
                            ld_pairs2(src + nt * 128, w[q][nt][0], w[q][nt][1]);
                            ld_pairs2(src + nt * 128 + 2, w[q][nt][2], w[q][nt][3]);
                        }
                    }
#pragma unroll
                for (int q = 0; q < BATCH; ++q)
                    if (need[q]) {
                        bool all = true;
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) all = all && (w[q][nt][e] >> 32) == 1ull;
                        if (all) need[q] = false;  // arrived: its words stay in w[q]
                        else miss = true;
                    }
                if (!__any_sync(0xffffffffu, miss)) break;
                __nanosleep(100);
                // warp-uniform decision: the votes above and below are executed by all 32 lanes
                if (__any_sync(0xffffffffu, clock64() - t0 > kWaitCycles || *abort_flag != 0)) {
                    failed = true;
                    break;
                }
            }
            if (failed) break;
#pragma unroll
            for (int q = 0; q < BATCH; ++q)
                if (j0 + q < cta) {
                    unsigned long long *src = p.pairs + (((size_t)(j0 + q) * 4 + warp) * MT) * 128 + lane * 4;
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) held[nt][e] += __uint_as_float((unsigned)w[q][nt][e]);
                        st_pairs2(src + nt * 128, 0ull, 0ull);  // ready for the next launch
                        st_pairs2(src + nt * 128 + 2, 0ull, 0ull);
                    }
                }
        }
        if (!failed) {
            if constexpr (EXCH) slab_push<MT>(p, ar, ar_epoch, held_b * 64 + warp * 16, g, t, held);
            else slab_store<MT>(p, held_b * 64 + warp * 16, g, t, held);
        } else {
            aborted = true;
            if (lane == 0) {
                *abort_flag = 1;
                atomicExch(p.status, QF_ERR_TIMEOUT);
            }
        }
    }
    if constexpr (EXCH) {
        // collect what this warp pushed: the row block finished last of all (the held one) and the full ones.
        // A tile that this warp could not finish (abort) is still counted, so that the call's epoch advances.
        const unsigned tiles_in_launch = (unsigned)(p.N >> 4);
        bool ok = !aborted;
        if (have_held) {
            if (ok) ok = slab_collect<MT>(p, ar, ar_epoch, held_b * 64 + warp * 16, g, t, abort_flag);
            if (lane == 0) exch_block_done(ar, ar_epoch, tiles_in_launch, !ok);
        }
        if (first_done >= 0)
            for (long long bb = first_done; bb <= last_done; ++bb) {
                if (ok) ok = slab_collect<MT>(p, ar, ar_epoch, bb * 64 + warp * 16, g, t, abort_flag);
                if (lane == 0) exch_block_done(ar, ar_epoch, tiles_in_launch, !ok);
            }
    }
}

template <bool BF16, int MT>
__global__ void __launch_bounds__(SLAB_THREADS, MT <= 2 ? 4 : 3) gemv_slab_kernel(const SlabParams p) {
    gemv_slab_body<BF16, MT, false>(p, NoExchange{});
}
template <bool BF16, int MT>
__global__ void __launch_bounds__(SLAB_THREADS, MT <= 2 ? 4 : 3)
gemv_slab_exch_kernel(const SlabParams p, const ArParams ar) {
    gemv_slab_body<BF16, MT, true>(p, ar);
}

// ---------------------------------------------------------------------------------------------
// prepack: canonical qweight + scales + zeros -> blob, and the inverse for the codes
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t slab_interleave_word(uint32_t w) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r |= ((w >> (8 * i)) & 0xFu) << (4 * i);            // even codes -> nibbles 0..3
        r |= ((w >> (8 * i + 4)) & 0xFu) << (4 * (i + 4));  // odd codes  -> nibbles 4..7
    }
    return r;
}
__device__ __forceinline__ uint32_t slab_deinterleave_word(uint32_t w) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r |= ((w >> (4 * i)) & 0xFu) << (8 * i);
        r |= ((w >> (4 * (i + 4))) & 0xFu) << (8 * i + 4);
    }
    return r;
}

// One thread per 32-bit word of the blob's code area (272 words per tile, the last 16 of them constants).
template <bool BF16, int ZMODE>
__global__ void __launch_bounds__(256) slab_prepack_kernel(const uint32_t *__restrict__ qw,
                                                           const uint16_t *__restrict__ scales,
                                                           const void *__restrict__ zeros, int zero_const,
                                                           uint32_t *__restrict__ blob, int64_t N, int64_t K,
                                                           int group) {
    const int64_t chunks = K >> 7;
    const int64_t tiles = (N >> 4) * chunks;
    const int64_t total = tiles * 272;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t tile = i / 272;
        const int w = (int)(i - tile * 272);
        const int64_t unit = tile >> 2;
        const int warp = (int)(tile & 3);
        const int64_t b = unit / chunks;
        const int64_t c = unit - b * chunks;
        const int64_t row0 = b * 64 + warp * 16;
        if (w < 256) {
            const int half = w >> 7;          // rows g or g + 8
            const int lane = (w >> 2) & 31;
            const int j = w & 3;
            const int64_t row = row0 + (lane >> 2) + 8 * half;
            const int64_t word = c * 16 + 4 * j + (lane & 3);
            blob[i] = slab_interleave_word(qw[row * (K >> 3) + word]);
        } else {
            const int64_t n = row0 + (w - 256);
            const int64_t gi = (c * 128) / group;
            const int z = load_zero<ZMODE>(zeros, zero_const, gi, n, N);
            const uint32_t zsub = BF16 ? int_to_bf16_bits(128 + z) : int_to_f16_bits(1024 + z);
            blob[i] = (zsub & 0xffffu) | ((uint32_t)scales[gi * N + n] << 16);
        }
    }
}

__global__ void __launch_bounds__(256) slab_unpack_kernel(const uint32_t *__restrict__ blob, uint32_t *__restrict__ qw,
                                                          int64_t N, int64_t K) {
    const int64_t chunks = K >> 7;
    const int64_t tiles = (N >> 4) * chunks;
    const int64_t total = tiles * 256;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t tile = i >> 8;
        const int w = (int)(i & 255);
        const int64_t unit = tile >> 2;
        const int warp = (int)(tile & 3);
        const int64_t b = unit / chunks;
        const int64_t c = unit - b * chunks;
        const int half = w >> 7;
        const int lane = (w >> 2) & 31;
        const int j = w & 3;
        const int64_t row = b * 64 + warp * 16 + (lane >> 2) + 8 * half;
        const int64_t word = c * 16 + 4 * j + (lane & 3);
        qw[row * (K >> 3) + word] = slab_deinterleave_word(blob[tile * 272 + w]);
    }
}

template <bool BF16>
static void slab_prepack_dispatch(int zmode, unsigned blocks, cudaStream_t s, const uint32_t *qw, const uint16_t *sc,
                                  const void *z, int zc, uint32_t *blob, int64_t N, int64_t K, int group) {
    if (zmode == QF_ZERO_CONST)
        slab_prepack_kernel<BF16, QF_ZERO_CONST><<<blocks, 256, 0, s>>>(qw, sc, z, zc, blob, N, K, group);
    else if (zmode == QF_ZERO_U4)
        slab_prepack_kernel<BF16, QF_ZERO_U4><<<blocks, 256, 0, s>>>(qw, sc, z, zc, blob, N, K, group);
    else
        slab_prepack_kernel<BF16, QF_ZERO_I8><<<blocks, 256, 0, s>>>(qw, sc, z, zc, blob, N, K, group);
}

int launch_slab_prepack(qf_ctx *ctx, const qf_linear_desc *d, const void *qw, const void *scales, const void *zeros,
                        void *blob, cudaStream_t s) {
    const int64_t total = (d->N / 16) * (d->K / 128) * 272;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    if (d->act_dtype == QF_BF16)
        slab_prepack_dispatch<true>(d->zero_mode, (unsigned)blocks, s, (const uint32_t *)qw, (const uint16_t *)scales,
                                    zeros, d->zero_const, (uint32_t *)blob, d->N, d->K, d->group_size);
    else
        slab_prepack_dispatch<false>(d->zero_mode, (unsigned)blocks, s, (const uint32_t *)qw, (const uint16_t *)scales,
                                     zeros, d->zero_const, (uint32_t *)blob, d->N, d->K, d->group_size);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

int launch_slab_unpack(qf_ctx *ctx, int64_t N, int64_t K, const void *blob, void *qw, cudaStream_t s) {
    const int64_t total = (N / 16) * (K / 128) * 256;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    slab_unpack_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint32_t *)blob, (uint32_t *)qw, N, K);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static size_t slab_smem_bytes(int depth, int m_pad) {
    return (size_t)depth * (2 * SLAB_UNIT_BYTES + m_pad * SLAB_X_PITCH) + 2 * (size_t)depth * 8 + 128 /*alignment*/;
}

int slab_m_pad(int64_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : M <= 16 ? 16 : 32; }

// Thread blocks per SM and ring depth for a launch. Small matrices: more, shorter thread blocks (every block's
// weights are in flight at once and there is room for the next kernel's blocks beside them); large ones: deep
// rings. QF_SLAB_CTAS / QF_SLAB_DEPTH in the environment override the heuristic (tuning).
void slab_geometry(int64_t M, int64_t N, int64_t K, int sm_count, int grid_request, int *grid_out, int *depth_out) {
    // read on every call (a tuning run changes them between launches); two getenv calls cost nothing next to a launch
    const char *e_ctas = std::getenv("QF_SLAB_CTAS");
    const char *e_depth = std::getenv("QF_SLAB_DEPTH");
    const int env_ctas = e_ctas ? std::atoi(e_ctas) : 0;
    const int env_depth = e_depth ? std::atoi(e_depth) : 0;
    const long long units = (N / 64) * (K / 128);
    const int m_pad = slab_m_pad(M);
    const size_t stage = 2 * SLAB_UNIT_BYTES + (size_t)m_pad * SLAB_X_PITCH;  // a pair of units
    // Measured on B200 (M = 1, bf16, CUDA-graph replays on weights that are not in L2; us per launch, 2 / 3 / 4
    // blocks per SM):   8.4 MB 4.8 / 6.0 / 6.2    17 MB 7.0 / 8.3 / 8.4    21 MB 8.3 / 10.1 / 9.8    29 MB 10.4 / 11.8 / 10.8
    //                   34 MB 11.3 / 13.1 / 11.5   42 MB 13.6 / 15.5 / 12.8  59 MB 17.9 / 20.5 / 16.4   235 MB 64 / 73 / 55.5
    // Large matrices want every warp slot streaming; small ones want room left on the SM, so that the next kernel of
    // the stream (programmatic dependent launch) is resident with its weights already in flight when this one ends.
    const long long wbytes = units * SLAB_UNIT_BYTES;
    int ctas = wbytes <= kSlabSmallBytes ? 2 : 4;
    if (m_pad > 16) ctas = std::min(ctas, 3);  // register budget of the four-batch-tile instantiation
    while (ctas > 1 && units / ((long long)sm_count * ctas) < 2) --ctas;
    if (env_ctas > 0) ctas = env_ctas;
    long long grid = (long long)sm_count * ctas;
    if (grid_request > 0) {
        // an explicit number of thread blocks (tests, tuning): any value works, an owner only waits for thread
        // blocks dispatched before it
        grid = grid_request;
        ctas = (int)std::min<long long>(4, std::max<long long>(1, (grid + sm_count - 1) / sm_count));
    }
    if (grid > units) grid = units;
    long long depth = (long long)((200u << 10) / ctas / stage);
    const long long per_max = ((units + grid - 1) / grid + 1) / 2;  // pairs a thread block streams
    if (depth > per_max) depth = per_max;
    if (depth > SLAB_MAX_DEPTH) depth = SLAB_MAX_DEPTH;
    // stages hold pairs of units; deeper rings measured equal or slower, shallow ones leave room on the SM
    // (30 MB: 3 stages 12.1 us, 4: 12.4, 5: 13.0; 235 MB: 59.5 / 59.1 / 59.1)
    const long long cap = wbytes <= (64ll << 20) ? 3 : 4;
    if (depth > cap) depth = cap;
    if (env_depth > 0) depth = env_depth;
    if (depth < 1) depth = 1;
    while (depth > 1 && slab_smem_bytes((int)depth, m_pad) > (size_t)(220u << 10)) --depth;
    *grid_out = (int)grid;
    *depth_out = (int)depth;
}

size_t slab_workspace_bytes(int grid, int64_t M) {
    const int mt = (slab_m_pad(M) + 7) / 8;
    return (size_t)grid * 4 * mt * 128 * sizeof(unsigned long long);
}

static bool slab_fixed_carveout() {
    const char *e = std::getenv("QF_SLAB_CARVEOUT");  // "0": leave the split to the driver (measurement)
    return !(e && e[0] == '0');
}

template <bool BF16, int MT>
static cudaError_t slab_set_attr() {
    cudaError_t e = cudaFuncSetAttribute(gemv_slab_kernel<BF16, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(220u << 10));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemv_slab_exch_kernel<BF16, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(220u << 10));
    // One shared-memory / L1 split for every launch of these kernels, whatever ring a launch asks for: the kernels
    // of a decode step follow each other under programmatic dependent launch, and thread blocks of the next kernel
    // only become resident beside the current one's if the SM does not have to be reconfigured in between (a
    // 70B-shaped step whose launches alternated between two splits ran 12 % slower than with one). The kernels
    // barely use L1: weights and activations arrive through bulk copies into shared memory.
    if (e == cudaSuccess && slab_fixed_carveout()) {
        e = cudaFuncSetAttribute(gemv_slab_kernel<BF16, MT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemv_slab_exch_kernel<BF16, MT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared);
    }
    return e;
}

int gemv_slab_init(qf_ctx *ctx) {
    QF_CUDA_TRY(ctx, (slab_set_attr<false, 1>()));
    QF_CUDA_TRY(ctx, (slab_set_attr<false, 2>()));
    QF_CUDA_TRY(ctx, (slab_set_attr<false, 4>()));
    QF_CUDA_TRY(ctx, (slab_set_attr<true, 1>()));
    QF_CUDA_TRY(ctx, (slab_set_attr<true, 2>()));
    QF_CUDA_TRY(ctx, (slab_set_attr<true, 4>()));
    return QF_OK;
}

static int launch_gemv_slab_impl(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X,
                                 const void *blob, void *Y, const void *residual, void *ws, cudaStream_t s,
                                 const ArParams *ar) {
    SlabParams p;
    p.blob = (const uint8_t *)blob;
    p.X = (const uint16_t *)X;
    p.Y = Y;
    p.residual = residual;
    p.pairs = (unsigned long long *)ws;
    p.status = ctx->dev_status;
    p.M = d->M;
    p.N = d->N;
    p.K = d->K;
    p.chunks = (int)(d->K / 128);
    p.units = (long long)(d->N / 64) * p.chunks;
    p.depth = plan.chunks_per_split;
    p.m_pad = slab_m_pad(d->M);
    p.out_dtype = d->out_dtype;
    p.epilogue = ar ? QF_EPI_NONE : d->epilogue;
    // QF_SLAB_STREAM_ONLY=1 (measurement only): the kernel moves every byte through its copy pipeline but converts
    // and multiplies nothing, so Y is NOT computed. It exists to time the ceiling the weight stream alone allows for
    // a given shape under the same launch sequence (graph, programmatic dependent launch) as the real kernel.
    const char *so = std::getenv("QF_SLAB_STREAM_ONLY");
    p.stream_only = (so && so[0] == '1') ? 1 : 0;
    const dim3 grid((unsigned)plan.split_k), blk(SLAB_THREADS);
    const size_t smem = slab_smem_bytes(p.depth, p.m_pad);
    const bool pdl = pdl_enabled();
    const int mt = (p.m_pad + 7) / 8;
    const bool bf = d->act_dtype == QF_BF16;
    cudaError_t le;
    if (ar) {
        // a thread block that collects waits for the peers' pushes while it holds its slot: the whole launch must be
        // resident at once on every rank
        int per_sm = 0;
        const void *fn = bf ? (mt == 1   ? (const void *)gemv_slab_exch_kernel<true, 1>
                               : mt == 2 ? (const void *)gemv_slab_exch_kernel<true, 2>
                                         : (const void *)gemv_slab_exch_kernel<true, 4>)
                            : (mt == 1   ? (const void *)gemv_slab_exch_kernel<false, 1>
                               : mt == 2 ? (const void *)gemv_slab_exch_kernel<false, 2>
                                         : (const void *)gemv_slab_exch_kernel<false, 4>);
        QF_CUDA_TRY(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, SLAB_THREADS, smem));
        if ((long long)per_sm * ctx->sm_count < (long long)grid.x)
            return fail(ctx, QF_ERR_UNSUPPORTED,
                        "an exchanging launch of " + std::to_string(grid.x) + " thread blocks is not resident at once (" +
                            std::to_string(per_sm) + " per SM fit)");
        if (bf)
            le = mt == 1   ? launch_kernel(gemv_slab_exch_kernel<true, 1>, grid, blk, smem, s, pdl, p, *ar)
                 : mt == 2 ? launch_kernel(gemv_slab_exch_kernel<true, 2>, grid, blk, smem, s, pdl, p, *ar)
                           : launch_kernel(gemv_slab_exch_kernel<true, 4>, grid, blk, smem, s, pdl, p, *ar);
        else
            le = mt == 1   ? launch_kernel(gemv_slab_exch_kernel<false, 1>, grid, blk, smem, s, pdl, p, *ar)
                 : mt == 2 ? launch_kernel(gemv_slab_exch_kernel<false, 2>, grid, blk, smem, s, pdl, p, *ar)
                           : launch_kernel(gemv_slab_exch_kernel<false, 4>, grid, blk, smem, s, pdl, p, *ar);
    } else if (bf) {
        le = mt == 1   ? launch_kernel(gemv_slab_kernel<true, 1>, grid, blk, smem, s, pdl, p)
             : mt == 2 ? launch_kernel(gemv_slab_kernel<true, 2>, grid, blk, smem, s, pdl, p)
                       : launch_kernel(gemv_slab_kernel<true, 4>, grid, blk, smem, s, pdl, p);
    } else {
        le = mt == 1   ? launch_kernel(gemv_slab_kernel<false, 1>, grid, blk, smem, s, pdl, p)
             : mt == 2 ? launch_kernel(gemv_slab_kernel<false, 2>, grid, blk, smem, s, pdl, p)
                       : launch_kernel(gemv_slab_kernel<false, 4>, grid, blk, smem, s, pdl, p);
    }
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, le);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

int launch_gemv_slab(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *blob, void *Y,
                     const void *residual, void *ws, cudaStream_t s) {
    return launch_gemv_slab_impl(ctx, d, plan, X, blob, Y, residual, ws, s, nullptr);
}

int launch_gemv_slab_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &plan, const void *X, const void *blob,
                        void *Y, void *ws, cudaStream_t s, const ArParams &ar) {
    return launch_gemv_slab_impl(ctx, d, plan, X, blob, Y, nullptr, ws, s, &ar);
}

}  // namespace qf
