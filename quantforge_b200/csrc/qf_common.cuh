// Shared device helpers and host-side context for the QuantForge B200 runtime.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>
#include <utility>
#include <vector>

#include "quantforge_rt.h"

namespace qf {

// ---------------------------------------------------------------------------------------------
// Host context
// ---------------------------------------------------------------------------------------------
struct TensorMapCacheEntry;

}  // namespace qf

struct qf_ctx {
    int device = 0;
    int sm_count = 148;
    std::string last_error;
    // Staging for the *_host entry points: two slots used in turn, so that the activations of call i+1 cross PCIe (on
    // the context's own copy stream) while the kernel of call i runs. Buffers only ever grow; a buffer that became
    // too small is kept until the context is destroyed (kernels enqueued earlier may still use it, and freeing
    // would synchronise the device in the middle of a hot call).
    struct HostSlot {
        void *x = nullptr;
        size_t x_bytes = 0;
        void *y = nullptr;
        size_t y_bytes = 0;
        cudaEvent_t copied_in = nullptr;   // activations of the slot's latest call are on the device
        cudaEvent_t kernel_done = nullptr; // its kernel has read them
    };
    HostSlot host_slot[2];
    int host_next = 0;
    cudaStream_t copy_stream = nullptr;
    std::vector<void *> retired;  // outgrown staging buffers
    // device status word written by kernels whose bounded waits expire (tcgen05 path)
    int *dev_status = nullptr;
    int *host_status = nullptr;  // pinned mirror
};

namespace qf {

extern std::atomic<long long> g_launch_count;

// Programmatic dependent launch (PDL): a kernel launched with it may start while the previous kernel in the
// stream is still draining; it must execute griddep_wait() before touching anything that kernel wrote.
// The linear kernels use the head start for what does not depend on the previous kernel: weight streams,
// converter constants, barrier and TMEM set-up. QF_PDL=0 in the environment turns it off.
bool pdl_enabled();
bool cluster_reduce_enabled();
// Largest launch of the tcgen05 kernel (2 blocks per SM) that runs as one wave of thread-block clusters: clusters
// are placed inside one GPC, which leaves block slots unused where the GPC's slot count is not a multiple of the
// cluster size (measured: 32 x 8, 80 x 3, 112 x 2 blocks fit; 48 x 6 = 288 of the 296 slots do not).
constexpr int kClusterMaxBlocks = 256;

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 bool pdl, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Same, with the grid grouped into thread-block clusters of `cluster` blocks ((1,1,1): no clusters).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                         bool pdl, dim3 cluster, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Makes `device` current for the lifetime of the object and restores the caller's device afterwards.
class DeviceGuard {
  public:
    explicit DeviceGuard(int device) {
        ok_ = cudaGetDevice(&prev_) == cudaSuccess;
        if (ok_ && prev_ != device) {
            ok_ = cudaSetDevice(device) == cudaSuccess;
            switched_ = ok_;
        }
    }
    ~DeviceGuard() {
        if (switched_) cudaSetDevice(prev_);
    }
    bool ok() const { return ok_; }
    DeviceGuard(const DeviceGuard &) = delete;
    DeviceGuard &operator=(const DeviceGuard &) = delete;

  private:
    int prev_ = -1;
    bool ok_ = false;
    bool switched_ = false;
};

inline int fail(qf_ctx *ctx, int status, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return status;
}

inline int cuda_fail(qf_ctx *ctx, cudaError_t e, const char *what) {
    return fail(ctx, QF_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// The compute entry points launch on the current device: it must be the context's.
inline int check_current_device(qf_ctx *ctx) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(ctx, QF_ERR_CUDA, "cudaGetDevice failed");
    if (dev != ctx->device)
        return fail(ctx, QF_ERR_BAD_ARG, "the current CUDA device (" + std::to_string(dev) +
                                             ") is not the context's device (" + std::to_string(ctx->device) + ")");
    return QF_OK;
}

#define QF_CUDA_TRY(ctx, expr)                                   \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) return cuda_fail(ctx, _e, #expr); \
    } while (0)

struct Plan {
    int path;            // QF_PATH_GEMV / QF_PATH_GEMM
    int split_k;         // number of K splits (slab GEMV: thread blocks of the launch)
    int chunks_per_split;  // GEMV: 128-code chunks per split; GEMM: k-blocks per split; slab GEMV: ring depth
    bool slab;           // QF_LAYOUT_GEMV_SLAB weights: the streaming GEMV kernel
    int m_tiles;         // GEMV: ceil(M/8); GEMM: batch tiles
    int bn;              // GEMM: batch tile width (MMA N)
    size_t ws_partial_bytes;
    size_t ws_counter_bytes;
};

// ---------------------------------------------------------------------------------------------
// Exchange over peer memory (row-parallel linears: partial outputs summed across GPUs inside the kernel)
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 8;
constexpr size_t kCommHeaderBytes = 256;  // epoch, done, padding

// Kernel-side view of a qf_comm. Every rank's buffer has the same layout:
//   epoch                          u32   calls completed on this comm (advanced by the last block of each call)
//   done                           u32   column blocks of the running call that have finished
//   slots [2][world][slot_elems]   (f32 value, u32 token) pairs, double-buffered by the parity of the epoch
// Slot [parity][src] of rank r is written by rank src only (peer stores) and read by rank r only.
// Why two buffers are enough: a rank starts call k+2 only after it finished call k+1, which needed every
// rank's pushes of call k+1, and a rank pushes for call k+1 only after its own call k (and its reads) finished.
struct ArParams {
    uint2 *slots[kMaxPeers];      // slots region of every rank's buffer (own rank: local address)
    uint2 *local_slots;           // = slots[rank]
    unsigned *epoch;              // local
    unsigned *done;               // local
    int *status;                  // device status word of the context (bounded waits report here)
    unsigned long long slot_elems;
    int world;
    int rank;
    int gather;                   // 0: Y[M, N] = sum over ranks; 1: Y[M, world*N], columns [r*N, (r+1)*N) from rank r
    long long wait_cycles;        // SM clocks a collect waits for the peers before it gives up (QF_ERR_TIMEOUT)
};

// Kernel argument of the exchange: an ArParams in the exchanging instantiations, an empty struct in the plain ones.
struct NoExchange {};
template <bool EXCH> struct ExchArg { typedef NoExchange type; };
template <> struct ExchArg<true> { typedef ArParams type; };

// Validates `d` and fills the launch plan. Returns QF_OK or an error status; `why` receives a message.
int make_plan(const qf_linear_desc *d, Plan *p, std::string *why);

// kernels (defined in their own translation units)
int launch_unpack(qf_ctx *ctx, const void *packed, void *out, int64_t rows, int64_t packed_cols, cudaStream_t s);
int launch_dequant(qf_ctx *ctx, const qf_linear_desc *d, const void *qw, const void *scales, const void *zeros,
                   void *w_out, cudaStream_t s);
int launch_gemv(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *qw,
                const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s);
int launch_gemm(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *qw,
                const void *scales, const void *zeros, void *Y, const void *residual, void *ws, cudaStream_t s);
int launch_prepack(qf_ctx *ctx, const void *in, void *out, int64_t n_words, int to_canonical, cudaStream_t s);
int launch_prepack_tiled(qf_ctx *ctx, const void *in, void *out, int64_t N, int64_t K, int to_canonical,
                         cudaStream_t s);
int gemm_block_k(int bn);
int launch_gemv_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *qw,
                   const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s, const ArParams &ar);
int launch_gemm_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *qw,
                   const void *scales, const void *zeros, void *Y, void *ws, cudaStream_t s, const ArParams &ar);
int launch_gemv_static(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *qw,
                       const void *scales, const void *zeros, void *Y, cudaStream_t s);
int gemv_init(qf_ctx *ctx);
int gemm_init(qf_ctx *ctx);
// streaming GEMV on QF_LAYOUT_GEMV_SLAB weights (qf_gemv_slab.cu)
int gemv_slab_init(qf_ctx *ctx);
// Blobs up to this size run with two thread blocks per SM, larger ones with four (see slab_geometry). Launched
// alone, matrices up to about 34 MB are faster with two (17 MB: 7.0 vs 8.4 us); inside a decode step, where the
// neighbours are kernels of other sizes, a limit of 36 MB measured no better than 16 MB (5.84 vs 5.79 ms per
// token on two GPUs), so the limit stays where the step-level numbers were taken.
constexpr long long kSlabSmallBytes = 16ll << 20;
int slab_m_pad(int64_t M);
void slab_geometry(int64_t M, int64_t N, int64_t K, int sm_count, int grid_request, int *grid_out, int *depth_out);
size_t slab_workspace_bytes(int grid, int64_t M);
int launch_gemv_slab(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *blob, void *Y,
                     const void *residual, void *ws, cudaStream_t s);
int launch_gemv_slab_ar(qf_ctx *ctx, const qf_linear_desc *d, const Plan &p, const void *X, const void *blob,
                        void *Y, void *ws, cudaStream_t s, const ArParams &ar);
int launch_slab_prepack(qf_ctx *ctx, const qf_linear_desc *d, const void *qw, const void *scales, const void *zeros,
                        void *blob, cudaStream_t s);
int launch_slab_unpack(qf_ctx *ctx, int64_t N, int64_t K, const void *blob, void *qw, cudaStream_t s);
int launch_repack_kn(qf_ctx *ctx, const void *w_kn, int packed_along_n, int64_t K, int64_t N, void *out,
                     cudaStream_t s);

// ---------------------------------------------------------------------------------------------
// Device helpers: nibble -> f16 / bf16 conversion with zero and scale applied in registers.
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// PDL: wait until the previous kernel of the stream has completed and its writes are visible (no-op without PDL).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// PDL: allow the next kernel of the stream to start its own independent prologue.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// 16-bit float bit patterns of small integers (exact in both formats for |v| <= 256).
__device__ __forceinline__ uint32_t int_to_f16_bits(int v) {
    return (uint32_t)__half_as_ushort(__int2half_rn(v));
}
__device__ __forceinline__ uint32_t int_to_bf16_bits(int v) {
    return __float_as_uint((float)v) >> 16;  // |v| <= 256 has <= 8 significant bits: exact
}
__device__ __forceinline__ uint32_t dup16(uint32_t h) { return h | (h << 16); }

// Per (row, group) constants for the converters below.
//   f16 : zsub = (1024 + z) x2, zfma = -(64 + z) x2      bf16: zsub = (128 + z) x2, zfma unused
template <bool BF16>
struct ZeroScale {
    uint32_t zsub, zfma, s2;
    __device__ __forceinline__ void set(int z, uint32_t scale_bits) {
        s2 = dup16(scale_bits & 0xffffu);
        if (BF16) {
            zsub = dup16(int_to_bf16_bits(128 + z));
            zfma = 0;
        } else {
            zsub = dup16(int_to_f16_bits(1024 + z));
            zfma = dup16(int_to_f16_bits(-(64 + z)));
        }
    }
};

// One packed word w holds codes c0..c7 (c_i = (w >> 4i) & 0xF).  Produces, in the activation type,
//   p[i] = ( (c_i - z) * s , (c_{i+4} - z) * s )   (low half, high half),  i = 0..3
// with the same roundings as `f16(sitofp(q)) - f16(sitofp(z))` (exact) followed by one
// round-to-nearest-even multiply (the reference's qf.dequant arithmetic).
//   f16 : (w & 0x000f000f) | 0x6400.. is 1024 + c  ;  (w & 0x00f000f0) | 0x6400.. is 1024 + 16c,
//         brought back by fma(v, 1/16, -(64 + z)) = c - z, exact.
//   bf16: ((w >> 4i) & 0x000f000f) | 0x4300.. is 128 + c.
template <bool BF16>
__device__ __forceinline__ void dequant8(uint32_t w, const ZeroScale<BF16> &zs, uint32_t (&p)[4]) {
    if (BF16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t v = lop3_and_or(w >> (4 * i), 0x000f000fu, 0x43004300u);
            p[i] = mul_bf16x2(sub_bf16x2(v, zs.zsub), zs.s2);
        }
    } else {
        const uint32_t w8 = w >> 8;
        uint32_t v0 = lop3_and_or(w, 0x000f000fu, 0x64006400u);
        uint32_t v1 = lop3_and_or(w, 0x00f000f0u, 0x64006400u);
        uint32_t v2 = lop3_and_or(w8, 0x000f000fu, 0x64006400u);
        uint32_t v3 = lop3_and_or(w8, 0x00f000f0u, 0x64006400u);
        p[0] = mul_f16x2(sub_f16x2(v0, zs.zsub), zs.s2);
        p[1] = mul_f16x2(fma_f16x2(v1, 0x2c002c00u, zs.zfma), zs.s2);
        p[2] = mul_f16x2(sub_f16x2(v2, zs.zsub), zs.s2);
        p[3] = mul_f16x2(fma_f16x2(v3, 0x2c002c00u, zs.zfma), zs.s2);
    }
}

// Zero point of (group gi, column n) for the three storage modes.
template <int ZMODE>
__device__ __forceinline__ int load_zero(const void *zeros, int zero_const, int64_t gi, int64_t n, int64_t N) {
    if (ZMODE == QF_ZERO_CONST) return zero_const;
    if (ZMODE == QF_ZERO_U4) {
        const uint32_t *z = reinterpret_cast<const uint32_t *>(zeros);
        return (int)((__ldg(z + gi * (N >> 3) + (n >> 3)) >> (4 * (int)(n & 7))) & 0xFu);
    }
    return (int)__ldg(reinterpret_cast<const int8_t *>(zeros) + gi * N + n);
}

__device__ __forceinline__ void store_out(void *Y, int out_dtype, int64_t idx, float v) {
    if (out_dtype == QF_F32) {
        reinterpret_cast<float *>(Y)[idx] = v;
    } else if (out_dtype == QF_F16) {
        reinterpret_cast<__half *>(Y)[idx] = __float2half_rn(v);
    } else {
        reinterpret_cast<__nv_bfloat16 *>(Y)[idx] = __float2bfloat16_rn(v);
    }
}

// Warp-level tensor-core MMA (m16n8k16, fp32 accumulate) and shared-memory loads used by the GEMV kernels.
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

__device__ __forceinline__ uint4 lds128g(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64g(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// ---------------------------------------------------------------------------------------------
// Thread-block clusters: barrier over all threads of all blocks of the cluster, and loads from a peer block's
// shared memory (distributed shared memory). QF_CLUSTER_REDUCE=0 in the environment keeps split-K on the
// global-memory path (partial tiles + arrival counters).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ float ld_dsmem_f1(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------------
// Cross-GPU exchange of finished output elements (device side). An element is pushed as an 8-byte
// (value, token) pair, written and read whole, so the pair itself says that it has arrived.
// ---------------------------------------------------------------------------------------------
constexpr long long kExchangeWaitCycles = 2000000000LL;  // about a second; then the kernel reports QF_ERR_TIMEOUT

__device__ __forceinline__ void st_pair_sys(uint2 *ptr, uint2 v) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(ptr), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2 *ptr) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned exch_read_epoch(const ArParams &ar) {
    unsigned e;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(ar.epoch) : "memory");
    return e;
}
__device__ __forceinline__ size_t exch_parity_offset(const ArParams &ar, unsigned epoch) {
    return (size_t)(epoch & 1u) * (size_t)ar.world * ar.slot_elems;
}
// Element `elem` (= m * N + n of this rank's output) of call `epoch` to every rank, own included.
__device__ __forceinline__ void exch_push(const ArParams &ar, unsigned epoch, size_t elem, float v) {
    const uint2 pair = make_uint2(__float_as_uint(v), epoch + 1u);
    const size_t off = exch_parity_offset(ar, epoch) + (size_t)ar.rank * ar.slot_elems + elem;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)  // unrolled: the pointer table stays in the kernel's parameter space
        if (r < ar.world) st_pair_sys(ar.slots[r] + off, pair);
}
// Two neighbouring elements (even n) as one 16-byte store / load; each 8-byte half is still written whole.
__device__ __forceinline__ void st_pair2_sys(uint2 *ptr, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_pair2_sys(const uint2 *ptr) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr)
                 : "memory");
    return v;
}
__device__ __forceinline__ void exch_push2(const ArParams &ar, unsigned epoch, size_t elem, float v0, float v1) {
    const uint4 pair2 = make_uint4(__float_as_uint(v0), epoch + 1u, __float_as_uint(v1), epoch + 1u);
    const size_t off = exch_parity_offset(ar, epoch) + (size_t)ar.rank * ar.slot_elems + elem;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < ar.world) st_pair2_sys(ar.slots[r] + off, pair2);
}
// Collects the tile rows [m0, m0+mrows) x columns [n0, n0+ncols) (ncols even; clipped to M and N) from every
// rank's slot and writes it out: the sum in rank order, or each rank's values into its own column range.
// A load from the slots costs a full L2 round trip, so each thread keeps U two-element units x W ranks in flight
// before it looks at any token, then polls (bounded) what has not arrived, again all at once. Returns false when a wait ran
// out or another thread already gave up.
template <int W, int U>
__device__ __forceinline__ bool exch_collect_tile_impl(const ArParams &ar, unsigned epoch, int64_t m0, int mrows,
                                                       int64_t n0, int ncols, int64_t M, int64_t N, void *Y,
                                                       int out_dtype, int tid, int nthreads, volatile int *fail) {
    const unsigned token = epoch + 1u;
    const uint2 *base = ar.local_slots + exch_parity_offset(ar, epoch);
    const int upr = ncols >> 1;  // 2-element units per row
    const int total = mrows * upr;
    const long long t0 = clock64();
    for (int u0 = tid; u0 < total; u0 += U * nthreads) {
        uint4 v[U][W];
        int64_t mm[U], nn[U];
        bool valid[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int u = u0 + j * nthreads;
            mm[j] = m0 + u / upr;
            nn[j] = n0 + 2 * (u % upr);
            valid[j] = u < total && mm[j] < M && nn[j] < N;
        }
#pragma unroll
        for (int j = 0; j < U; ++j)
#pragma unroll
            for (int r = 0; r < W; ++r)
                if (valid[j] && r < ar.world)
                    v[j][r] = ld_pair2_sys(base + (size_t)r * ar.slot_elems + (size_t)(mm[j] * N + nn[j]));
        // poll what has not arrived, all missing units at once (one round trip per round, not per unit)
        while (true) {
            bool miss = false;
#pragma unroll
            for (int j = 0; j < U; ++j)
#pragma unroll
                for (int r = 0; r < W; ++r)
                    if (valid[j] && r < ar.world && (v[j][r].y != token || v[j][r].w != token)) miss = true;
            if (!miss) break;
            __nanosleep(100);
            if (clock64() - t0 > ar.wait_cycles || *fail) return false;
#pragma unroll
            for (int j = 0; j < U; ++j)
#pragma unroll
                for (int r = 0; r < W; ++r)
                    if (valid[j] && r < ar.world && (v[j][r].y != token || v[j][r].w != token))
                        v[j][r] = ld_pair2_sys(base + (size_t)r * ar.slot_elems + (size_t)(mm[j] * N + nn[j]));
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (!valid[j]) continue;
            if (ar.gather) {
                const int64_t row = mm[j] * (N * ar.world) + nn[j];
#pragma unroll
                for (int r = 0; r < W; ++r)
                    if (r < ar.world) {
                        store_out(Y, out_dtype, row + (int64_t)r * N, __uint_as_float(v[j][r].x));
                        store_out(Y, out_dtype, row + (int64_t)r * N + 1, __uint_as_float(v[j][r].z));
                    }
            } else {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int r = 0; r < W; ++r)
                    if (r < ar.world) {
                        s0 += __uint_as_float(v[j][r].x);
                        s1 += __uint_as_float(v[j][r].z);
                    }
                store_out(Y, out_dtype, mm[j] * N + nn[j], s0);
                store_out(Y, out_dtype, mm[j] * N + nn[j] + 1, s1);
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool exch_collect_tile(const ArParams &ar, unsigned epoch, int64_t m0, int mrows, int64_t n0,
                                                  int ncols, int64_t M, int64_t N, void *Y, int out_dtype, int tid,
                                                  int nthreads, volatile int *fail) {
    if (ar.world <= 2)
        return exch_collect_tile_impl<2, 8>(ar, epoch, m0, mrows, n0, ncols, M, N, Y, out_dtype, tid, nthreads, fail);
    if (ar.world <= 4)
        return exch_collect_tile_impl<4, 4>(ar, epoch, m0, mrows, n0, ncols, M, N, Y, out_dtype, tid, nthreads, fail);
    return exch_collect_tile_impl<8, 2>(ar, epoch, m0, mrows, n0, ncols, M, N, Y, out_dtype, tid, nthreads, fail);
}
// One thread per finished block, after the block's collects: the last block of the launch advances the epoch.
__device__ __forceinline__ void exch_block_done(const ArParams &ar, unsigned epoch, unsigned blocks_in_launch,
                                                bool failed) {
    if (failed) atomicExch(ar.status, QF_ERR_TIMEOUT);
    __threadfence();
    if (atomicAdd(ar.done, 1u) == blocks_in_launch - 1u) {
        *ar.done = 0u;
        unsigned next = epoch + 1u;
        if (next == 0xFFFFFFFFu) next = 1u;  // its token would be 0, the value of never-written memory
        *ar.epoch = next;
    }
}

#endif  // __CUDACC__

}  // namespace qf
