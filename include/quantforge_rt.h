/*
 * quantforge_rt.h - C ABI of the B200 (sm_100a) runtime for QuantForge's W4A16 hot path.
 *
 * The QuantForge reference is an MLIR dialect (ops qf.unpack, qf.dequant) plus passes that
 * lower those ops to arithmetic; it ships no runtime.  This library is the runtime those ops
 * lower INTO: each entry point below replaces the lowering (or the PyTorch statement) of one
 * reference op, cited beside it by its path inside the reference project.
 *
 * Conventions
 *   - every function returns a qf_status (0 = QF_OK, negative = error); no exception crosses the ABI;
 *   - the caller owns every buffer; pointers are DEVICE pointers unless a name ends in `_host`;
 *     device buffers must be 16-byte aligned;
 *   - launches are asynchronous on the `stream` argument (a cudaStream_t passed as void*; NULL = default stream);
 *   - the hot calls allocate nothing: split-K scratch comes from the caller (`workspace`);
 *   - there is no CPU fallback: without a CUDA device every compute call returns QF_ERR_CUDA.
 *
 * Canonical tensor layouts for a linear Y[M,N] = X[M,K] . W^T, group size g, G = K/g
 *   qweight  int8[N, K/2] == little-endian uint32[N, K/8]; nibble i of word j of row n is code q[n, 8j+i]
 *   scales   f16|bf16 [G, N]   (same 16-bit type as the activations)
 *   qzeros   QF_ZERO_U4 : uint32[G, N/8], 8 four-bit codes per word along N, LSB first
 *            QF_ZERO_I8 : int8[G, N] (signed, the dialect's zero_point element type)
 *            QF_ZERO_CONST : no tensor, the value desc.zero_const
 *   X        f16|bf16 [M, K] row-major,  Y f16|bf16|f32 [M, N] row-major
 */
#ifndef QUANTFORGE_RT_H
#define QUANTFORGE_RT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QF_RT_VERSION 100 /* major*10000 + minor*100 + patch */

typedef enum qf_status {
    QF_OK = 0,
    QF_ERR_BAD_ARG = -1,       /* null / misaligned pointer, shape not a multiple of the tile */
    QF_ERR_UNSUPPORTED = -2,   /* valid request the kernels do not cover (e.g. group size) */
    QF_ERR_CUDA = -3,          /* a CUDA runtime/driver call failed; see qf_last_error */
    QF_ERR_NCCL = -4,
    QF_ERR_TIMEOUT = -5,       /* a bounded device-side wait expired */
    QF_ERR_UNIMPLEMENTED = -6,
    QF_ERR_WORKSPACE = -7      /* workspace missing or smaller than qf_w4a16_workspace_bytes */
} qf_status;

typedef enum qf_dtype { QF_F16 = 0, QF_BF16 = 1, QF_F32 = 2 } qf_dtype;
typedef enum qf_zero_mode { QF_ZERO_CONST = 0, QF_ZERO_U4 = 1, QF_ZERO_I8 = 2 } qf_zero_mode;

/* Which kernel family serves a linear.  AUTO: M <= 2 -> GEMV kernel unless the weight matrix is large (32 MB
 * prepacked, 40 MB canonical), M >= 3 -> tcgen05 GEMM kernel (measured crossovers on B200); prepacked weights
 * (QF_LAYOUT_GEMV_SLAB always runs the streaming GEMV kernel, the other prepacked layouts the tcgen05 kernel),
 * N % 128 != 0 and a fused epilogue override it, see qf_w4a16_plan. */
typedef enum qf_path { QF_PATH_AUTO = 0, QF_PATH_GEMV = 1, QF_PATH_GEMM = 2 } qf_path;

/*
 * Order of the eight 4-bit codes inside each 32-bit word of qweight.
 *   QF_LAYOUT_CANONICAL   : nibble i holds code 8j+i (what qf.unpack defines; lib/Transforms/LowerUnpackToNVVM.cpp:254-265)
 *   QF_LAYOUT_INTERLEAVED : nibbles hold codes 8j + {0,2,4,6,1,3,5,7}; produced once by qf_prepack_w4. With it the
 *                           lop3 converter yields (k, k+1) pairs directly and the GEMM kernel skips a byte permute.
 *                           Rows and words per row are unchanged: a pure permutation inside each word.
 *   QF_LAYOUT_TILED       : INTERLEAVED words regrouped so that the 128 rows x 128 codes (8 KB) a thread block
 *                           consumes per pipeline step are contiguous in HBM: word w (0..15) of row r (0..127) of
 *                           k-block kb of row tile nt sits at word index ((nt * K/128 + kb) * 128 + r) * 16 + w.
 *                           Needs N % 128 == 0. Produced once by qf_prepack_w4_tiled.
 *   QF_LAYOUT_GEMV_SLAB   : one blob that holds codes, scales and zeros in the order the streaming GEMV kernel
 *                           consumes them, so that every thread block reads ONE contiguous range of HBM with bulk
 *                           copies. Unit u = b * (K/128) + c covers weight rows [64b, 64b+64) x codes [128c, 128c+128)
 *                           and is QF_SLAB_UNIT_BYTES long: four tiles (16 rows each) of
 *                             512 B  rows r = 0..7 : lane (r, t) owns the interleaved words t, t+4, t+8, t+12 of the chunk
 *                             512 B  rows r + 8    : same
 *                              64 B  per row: 16-bit converter constant (magic + zero point) | 16-bit scale << 16
 *                           `qweight` of the linear calls points to the blob; `scales` and `qzeros` are ignored (may be
 *                           NULL). The blob is specific to (group_size, act_dtype, zero mode) of the descriptor it was
 *                           built with. Needs N % 64 == 0; serves M <= QF_SLAB_MAX_M. Produced by qf_prepack_gemv_slab.
 */
typedef enum qf_weight_layout {
    QF_LAYOUT_CANONICAL = 0,
    QF_LAYOUT_INTERLEAVED = 1,
    QF_LAYOUT_TILED = 2,
    QF_LAYOUT_GEMV_SLAB = 3
} qf_weight_layout;
#define QF_SLAB_UNIT_BYTES 4352
#define QF_SLAB_MAX_M 32

/*
 * Work fused behind the contraction (no counterpart in the reference, whose furthest fusion is unpack + dequant,
 * lib/Transforms/FuseUnpackDequant.cpp:68-305; these remove the elementwise kernels that follow the linears of a
 * decoder layer).
 *   QF_EPI_SILU_MUL     : gate and up projections as ONE linear whose weight rows alternate in groups of 8:
 *                         rows [16j, 16j+8) = gate rows [8j, 8j+8), rows [16j+8, 16j+16) = up rows [8j, 8j+8)
 *                         (scales and zeros permuted alike); desc.N counts both (a multiple of 16). The kernel
 *                         writes Y[M, N/2] = silu(gate) * up, silu(v) = v / (1 + exp(-v)), evaluated in fp32 on the
 *                         fp32 accumulators and rounded once.
 *   QF_EPI_RESIDUAL_ADD : Y[M, N] = X . W^T + R, R [M, N] in out_dtype (the `residual` argument of
 *                         qf_w4a16_linear_fused; R may alias Y), added in fp32 before the one rounding.
 * Served by the streaming GEMV kernel (QF_LAYOUT_GEMV_SLAB) and by the tcgen05 kernel.
 */
typedef enum qf_epilogue { QF_EPI_NONE = 0, QF_EPI_SILU_MUL = 1, QF_EPI_RESIDUAL_ADD = 2 } qf_epilogue;

typedef struct qf_ctx qf_ctx;

typedef struct qf_linear_desc {
    int64_t M, N, K;
    int32_t group_size;  /* multiple of 128 dividing K (K itself = per-output-channel) */
    int32_t act_dtype;   /* qf_dtype of X and of scales: QF_F16 or QF_BF16 */
    int32_t out_dtype;   /* qf_dtype of Y */
    int32_t zero_mode;   /* qf_zero_mode */
    int32_t zero_const;  /* used when zero_mode == QF_ZERO_CONST (8 = symmetric int4, 0 = the zp==0 fast path) */
    int32_t path;        /* qf_path */
    int32_t split_k;     /* 0 = heuristic; >0 requests a number of K splits (clamped to what the kernel can run;
                            qf_w4a16_plan reports the split in use). With QF_LAYOUT_GEMV_SLAB: the number of
                            thread blocks the weight stream is divided among (0 = a multiple of the SM count). */
    int32_t weight_layout; /* qf_weight_layout of qweight */
    int32_t epilogue;    /* qf_epilogue */
    int32_t reserved[3]; /* must be zero */
} qf_linear_desc;

int qf_version(void);
const char *qf_status_string(int status);

/* One context per device. Owns only small caches (tensor maps, staging buffers of the *_host calls). */
int qf_ctx_create(qf_ctx **out, int device);
int qf_ctx_destroy(qf_ctx *ctx);
/* Message of the last error recorded on this context (never NULL). */
const char *qf_last_error(const qf_ctx *ctx);

/*
 * qf.unpack  (include/QuantForge/Dialect/QuantForge/QuantForgeOps.td:18-42; arithmetic:
 * lib/Transforms/LowerUnpackToArith.cpp:173-214, word order lib/Transforms/LowerUnpackToNVVM.cpp:221-280;
 * python/quantforge/baseline.py:34-49 `unpack_int4`).
 * packed int8[rows, packed_cols] -> out int8[rows, 2*packed_cols]:
 * out[r, 2i] = b & 0xF, out[r, 2i+1] = (b >>logical 4) & 0xF.  Bit-exact.
 */
int qf_unpack_int4(qf_ctx *ctx, const void *packed_i8, void *out_i8, int64_t rows, int64_t packed_cols, void *stream);

/*
 * qf.dequant(qf.unpack(w))  materialised (the fused elementwise op of
 * lib/Transforms/FuseUnpackDequant.cpp:209-304; dequant arithmetic
 * lib/Transforms/LowerDequantToArith.cpp:141-159; zp==0 path
 * lib/Transforms/CanonicalizeDequantZeroPoint.cpp:177-192).
 * W[n,k] = round_act((q[n,k] - z[k/g,n]) * s[k/g,n]) written as act_dtype [N,K].
 * Uses N, K, group_size, act_dtype, zero_mode, zero_const of `desc`.  The linear below never
 * materialises W; this entry point exists because the reference op does and to make the
 * in-register conversion testable bit for bit.
 */
int qf_dequant_w4(qf_ctx *ctx, const qf_linear_desc *desc, const void *qweight, const void *scales,
                  const void *qzeros_or_null, void *w_out, void *stream);

/*
 * linalg.matmul(x, qf.dequant(qf.unpack(w), scale, zp))  as one call
 * (matcher lib/Transforms/ConvertLinalgToQuantForge.cpp:63-209, contraction :185-203;
 * python/quantforge/baseline.py:52-72 `gemv_int4_baseline`).
 * fp32 accumulation.  `workspace` must hold qf_w4a16_workspace_bytes(desc) bytes, be zero-filled
 * once before its first use, and not be shared by calls that overlap in time; the kernels leave
 * it ready for the next call.  It may be NULL when the size is 0.
 */
size_t qf_w4a16_workspace_bytes(const qf_linear_desc *desc);
int qf_w4a16_linear(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight, const void *scales,
                    const void *qzeros_or_null, void *Y, void *workspace, size_t workspace_bytes, void *stream);

/*
 * The linear with a fused epilogue (desc->epilogue, see qf_epilogue). `residual` is read only by
 * QF_EPI_RESIDUAL_ADD and may be NULL otherwise. With QF_EPI_NONE this is qf_w4a16_linear.
 */
int qf_w4a16_linear_fused(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight,
                          const void *scales, const void *qzeros_or_null, void *Y, const void *residual,
                          void *workspace, size_t workspace_bytes, void *stream);

/*
 * `count` linears enqueued back to back on `stream` by one call (the linears of a decoder layer: q/k/v as one
 * concatenated linear, o with the residual, gate/up with SiLU * mul, down with the residual). Entry i uses
 * descs[i], X[i], qweight[i], scales[i], qzeros[i] (may be NULL), Y[i], residual[i] (`residual` itself may be
 * NULL). Consecutive kernels are chained with programmatic dependent launch, so entry i+1 may read what entry i
 * wrote. `workspace` must hold the largest qf_w4a16_workspace_bytes over the entries. Stops at the first entry
 * that fails and returns its status (earlier entries stay enqueued).
 */
int qf_w4a16_linear_batched(qf_ctx *ctx, int count, const qf_linear_desc *descs, const void *const *X,
                            const void *const *qweight, const void *const *scales, const void *const *qzeros,
                            void *const *Y, const void *const *residual, void *workspace, size_t workspace_bytes,
                            void *stream);

/*
 * The same linear for callers that hold activations in HOST memory (the reference's Python entry
 * point takes CPU tensors when no GPU is used): copies X_host to the device, runs the kernel,
 * copies Y back and waits.  Weights, scales and zeros stay DEVICE pointers (they are loaded once).
 * Staging buffers live in the context and grow on first use; workspace as above.
 */
int qf_w4a16_linear_host(qf_ctx *ctx, const qf_linear_desc *desc, const void *X_host, const void *qweight,
                         const void *scales, const void *qzeros_or_null, void *Y_host, void *workspace,
                         size_t workspace_bytes, void *stream);
/*
 * The same without the final wait: the copies and the kernel are enqueued on `stream` and the call returns.
 * Y_host holds the result once the caller has synchronised `stream`; X_host must stay unchanged until then.
 * Use page-locked host buffers (with pageable ones the copies block the host anyway). Calls on one stream may be
 * issued back to back: the context keeps two staging slots and copies the activations of a call on a stream of its
 * own, so that they cross PCIe while the previous call's kernel runs; results return on `stream`. The slot written by
 * call i+2 holds Y of call i until that call's copy back has been enqueued on `stream`, which stream order guarantees.
 * Calls on different streams of one context must not overlap. Staging grows on first use of a larger shape
 * (a device allocation); outgrown buffers are released with the context.
 */
int qf_w4a16_linear_host_async(qf_ctx *ctx, const qf_linear_desc *desc, const void *X_host, const void *qweight,
                         const void *scales, const void *qzeros_or_null, void *Y_host, void *workspace,
                         size_t workspace_bytes, void *stream);

/*
 * One-time weight prepack: canonical -> QF_LAYOUT_INTERLEAVED (or back with to_canonical != 0).
 * n_words = N * K / 8 32-bit words; in and out may alias. The inverse of the permutation exists so that
 * unpack(prepack^-1(prepack(w))) == unpack(w) can be checked bit for bit. No reference counterpart: the
 * reference never fixes a device weight layout (its packing helper is python/quantforge/baseline.py:17-31).
 */
int qf_prepack_w4(qf_ctx *ctx, const void *qweight_in, void *qweight_out, int64_t n_words, int to_canonical,
                  void *stream);
/* canonical [N, K/8] words -> QF_LAYOUT_TILED (or back with to_canonical != 0). in and out must not alias. */
int qf_prepack_w4_tiled(qf_ctx *ctx, const void *qweight_in, void *qweight_out, int64_t N, int64_t K,
                        int to_canonical, void *stream);

/*
 * Bytes of a weight tensor of N rows x K codes in `layout`: N*K/2 for the canonical, interleaved and tiled layouts
 * (pure permutations), (N/64)*(K/128)*QF_SLAB_UNIT_BYTES for QF_LAYOUT_GEMV_SLAB (scales and zeros included).
 * 0 when the layout does not admit the shape.
 */
size_t qf_prepack_bytes(int layout, int64_t N, int64_t K);

/*
 * One-time prepack for the streaming GEMV kernel: canonical qweight + scales + zeros -> one QF_LAYOUT_GEMV_SLAB
 * blob of qf_prepack_bytes(QF_LAYOUT_GEMV_SLAB, N, K) bytes (16-byte aligned, must not alias the inputs).
 * Uses N, K, group_size, act_dtype, zero_mode, zero_const of `desc`. No reference counterpart (see qf_prepack_w4).
 * qf_unpack_gemv_slab writes the codes of a blob back as canonical qweight [N, K/2]: the inverse permutation,
 * there so that prepacking can be checked bit for bit.
 */
int qf_prepack_gemv_slab(qf_ctx *ctx, const qf_linear_desc *desc, const void *qweight, const void *scales,
                         const void *qzeros_or_null, void *blob_out, void *stream);
int qf_unpack_gemv_slab(qf_ctx *ctx, int64_t N, int64_t K, const void *blob, void *qweight_out, void *stream);

/*
 * Weight orientation of the reference's compiler half: its matcher puts the quantised operand of linalg.matmul
 * as W[K, N] (lib/Transforms/ConvertLinalgToQuantForge.cpp:185-203) and its tests pack two codes per byte along
 * the LAST dim, i.e. along N (test/Transforms/lower_unpack_to_arith.mlir:31-35). The kernels contract over rows
 * packed along K (python/quantforge/baseline.py:58-71). This converts once, on the device:
 *   packed_along_n = 0 : w_kn is int8[K, N], one code (0..15, upper bits ignored) per byte
 *   packed_along_n = 1 : w_kn is int8[K, N/2], byte j of row k = code[k, 2j] | code[k, 2j+1] << 4
 * -> qweight_out int8[N, K/2] canonical. K % 8 == 0, N % 2 == 0.
 */
int qf_repack_kn_to_canonical(qf_ctx *ctx, const void *w_kn, int packed_along_n, int64_t K, int64_t N,
                              void *qweight_out, void *stream);

/*
 * Sticky device-side status of this context: QF_OK, or QF_ERR_TIMEOUT when a kernel's bounded wait expired
 * (the kernel then returned without finishing its tile). Reading it does not synchronise; call it after the
 * stream has been synchronised. qf_ctx_clear_status resets it.
 */
int qf_ctx_status(const qf_ctx *ctx);
int qf_ctx_clear_status(qf_ctx *ctx);

/*
 * The GEMV-kernel linear for callers that must not allocate device memory and have no scratch buffer to lend.
 * (No counterpart in the reference, which has no runtime and therefore no memory policy.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits - inside a host framework that owns the whole
 * device heap and hands plugins raw tensors only, in a latency-critical serving loop where an allocation would
 * synchronise the device, or in a process started with a fixed memory budget that is already spent on weights.
 * Such callers cannot provide the split-K `workspace` of qf_w4a16_linear either.
 *
 * This entry point runs the same kernel as qf_w4a16_linear with path = QF_PATH_GEMV, but its split-K partial
 * sums and arrival counters live in a scratch array that is part of the library image: a file-scope
 * `static __device__` array of QF_STATIC_SCRATCH_BYTES (16 MiB) that every GPU loading the library holds until
 * the process exits. The call issues no cudaMalloc / cudaFree and calls no allocating library routine.
 * (Plans that sum their splits inside a thread-block cluster - 2..8 short splits - use no scratch at all; the
 * array then only has its counters cleared.)
 *   - Limits: a linear whose plan needs more scratch than the array holds is refused with QF_ERR_WORKSPACE
 *     (the message names both sizes); use qf_w4a16_linear with your own workspace for those. For K <= 4096
 *     desc.split_k = 1 is a plan without any scratch; longer K is always split (a split covers at most 4096
 *     codes), so the request is clamped, see qf_w4a16_plan.
 *   - The array is shared by every call on that device and keeps the previous call's contents. The counters a
 *     call uses are cleared on `stream` before the kernel starts; the partial sums are fully overwritten before
 *     they are read. Two calls that overlap in time on one device (different streams, or different host threads)
 *     race on the array: serialise them.
 *   - The first call on each device looks up the array's device address and raises the kernel's shared-memory
 *     limit. Make that first call outside any stream capture.
 * `ctx` may be NULL; when given it only receives the error message.
 */
#define QF_STATIC_SCRATCH_BYTES (16u << 20)
int qf_w4a16_gemv_static_scratch(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight,
                                 const void *scales, const void *qzeros_or_null, void *Y, void *stream);

/*
 * Tensor-parallel linears with the cross-GPU step inside the kernel. (No counterpart in the reference, which runs
 * on one device; the multi-GPU deployment this runtime adds would otherwise follow each linear with an NCCL
 * all-reduce or all-gather.) One process per GPU of one node, up to 8 ranks.
 *
 * qf_w4a16_linear_allreduce  row-parallel: each rank holds the K shard [rank*K/world, (rank+1)*K/world) of the
 *   weights, scales and zeros and the matching columns of X; `desc->K` is the shard's K. Every rank receives
 *   the full sum in its own Y[M, N], bit-identical on all ranks (fp32 partial outputs summed in rank order,
 *   then rounded once).
 * qf_w4a16_linear_allgather  column-parallel: each rank holds the output-column shard [rank*N, (rank+1)*N) of the
 *   weights (`desc->N` is the shard's N, the same on every rank) and the whole X. Every rank receives the whole
 *   output in its own Y[M, world*N]; columns [r*N, (r+1)*N) come from rank r.
 *
 * Both serve desc->M <= 64 (decode batches; beyond that the exchange is bandwidth-bound on the links and a bulk
 * collective after qf_w4a16_linear is the better tool) on either kernel, as qf_w4a16_linear would choose it.
 * The block that finishes a tile of the output pushes it into all ranks' exchange buffers with peer stores over
 * NVLink (value and arrival token in one 8-byte store) and polls for the other ranks' pushes of the same tile,
 * so the exchange overlaps the weight streams still running and no separate collective is launched.
 *
 * Set-up, once per group of ranks:
 *   qf_comm_create(ctx, rank, world, max_out_elems, &comm)   allocates this rank's exchange buffer
 *                                                            (16 * world * max_out_elems bytes + 256)
 *   qf_comm_export(comm, handle)                             QF_COMM_HANDLE_BYTES bytes to send to every rank
 *   qf_comm_connect(comm, handles, world)                    handles of all ranks, in rank order; maps the peers
 *   <a barrier of the caller's own, e.g. torch.distributed.barrier()>  before the first call
 * and a barrier again before qf_comm_destroy. world == 1 needs no handles (connect may be skipped).
 * Rules: all ranks make the same sequence of calls on a comm (any mix of shapes and of the two entry points);
 * calls on one comm are stream-ordered on each rank (one stream, or serialised); desc->M * desc->N <=
 * max_out_elems. A rank that waits longer than about a second for a peer gives up: its Y is incomplete,
 * qf_ctx_status(ctx) reads QF_ERR_TIMEOUT after the stream is synchronised, and the comm must be destroyed.
 * `workspace` as for qf_w4a16_linear with the same desc. After 2^32 - 2 calls on one comm the arrival token
 * repeats; an element that no call has written for that long could then be taken for arrived.
 */
typedef struct qf_comm qf_comm;
#define QF_COMM_HANDLE_BYTES 64
int qf_comm_create(qf_ctx *ctx, int rank, int world, size_t max_out_elems, qf_comm **out);
int qf_comm_export(const qf_comm *comm, void *handle_out);
int qf_comm_connect(qf_comm *comm, const void *handles, int n_handles);
int qf_comm_destroy(qf_comm *comm);
int qf_w4a16_linear_allreduce(qf_ctx *ctx, qf_comm *comm, const qf_linear_desc *desc, const void *X,
                              const void *qweight, const void *scales, const void *qzeros_or_null, void *Y,
                              void *workspace, size_t workspace_bytes, void *stream);
int qf_w4a16_linear_allgather(qf_ctx *ctx, qf_comm *comm, const qf_linear_desc *desc, const void *X,
                              const void *qweight, const void *scales, const void *qzeros_or_null, void *Y,
                              void *workspace, size_t workspace_bytes, void *stream);

/* Which kernel family `desc` resolves to (QF_PATH_GEMV / QF_PATH_GEMM) and the K split it will use. */
int qf_w4a16_plan(const qf_linear_desc *desc, int32_t *path_out, int32_t *split_k_out);

/* Number of kernel launches this library has enqueued since it was loaded (all contexts). */
int64_t qf_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* QUANTFORGE_RT_H */
