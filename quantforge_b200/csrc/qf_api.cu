// C ABI of the runtime (include/quantforge_rt.h): argument checks, planning, dispatch.
#include <cstdlib>
#include <cstring>
#include <new>

#include "qf_common.cuh"

namespace qf {

std::atomic<long long> g_launch_count{0};

bool pdl_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("QF_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

bool cluster_reduce_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("QF_CLUSTER_REDUCE");
        return !(e && e[0] == '0');
    }();
    return on;
}

static constexpr int kSmCount = 148;  // planning constant: the library targets B200 only
// The split-K arrival counters occupy a FIXED region at the start of the workspace, so that a
// workspace reused by linears of different shapes never exposes stale partial sums as counters.
static constexpr int kMaxCounters = 16384;
static constexpr size_t kCounterBytes = (size_t)kMaxCounters * sizeof(int);

static bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

int make_plan(const qf_linear_desc *d, Plan *p, std::string *why) {
    auto bad = [&](int st, const char *m) {
        if (why) *why = m;
        return st;
    };
    if (!d) return bad(QF_ERR_BAD_ARG, "desc is null");
    if (d->M < 0 || d->N <= 0 || d->K <= 0) return bad(QF_ERR_BAD_ARG, "M, N, K must be positive (M may be 0)");
    if (d->K % 128 != 0) return bad(QF_ERR_BAD_ARG, "K must be a multiple of 128");
    if (d->N % 16 != 0) return bad(QF_ERR_BAD_ARG, "N must be a multiple of 16");
    if (d->group_size <= 0 || d->group_size % 128 != 0 || d->K % d->group_size != 0)
        return bad(QF_ERR_UNSUPPORTED, "group_size must be a multiple of 128 that divides K");
    if (d->act_dtype != QF_F16 && d->act_dtype != QF_BF16)
        return bad(QF_ERR_UNSUPPORTED, "act_dtype must be QF_F16 or QF_BF16");
    if (d->out_dtype != QF_F16 && d->out_dtype != QF_BF16 && d->out_dtype != QF_F32)
        return bad(QF_ERR_UNSUPPORTED, "out_dtype must be QF_F16, QF_BF16 or QF_F32");
    if (d->zero_mode != QF_ZERO_CONST && d->zero_mode != QF_ZERO_U4 && d->zero_mode != QF_ZERO_I8)
        return bad(QF_ERR_BAD_ARG, "unknown zero_mode");
    if (d->zero_mode == QF_ZERO_CONST && (d->zero_const < -128 || d->zero_const > 127))
        return bad(QF_ERR_BAD_ARG, "zero_const must fit a signed 8-bit zero point");
    if (d->split_k < 0) return bad(QF_ERR_BAD_ARG, "split_k must be >= 0");
    if (d->weight_layout != QF_LAYOUT_CANONICAL && d->weight_layout != QF_LAYOUT_INTERLEAVED &&
        d->weight_layout != QF_LAYOUT_TILED && d->weight_layout != QF_LAYOUT_GEMV_SLAB)
        return bad(QF_ERR_BAD_ARG, "unknown weight_layout");
    if (d->epilogue != QF_EPI_NONE && d->epilogue != QF_EPI_SILU_MUL && d->epilogue != QF_EPI_RESIDUAL_ADD)
        return bad(QF_ERR_BAD_ARG, "unknown epilogue");
    for (int i = 0; i < 3; ++i)
        if (d->reserved[i] != 0) return bad(QF_ERR_BAD_ARG, "reserved fields must be zero");
    p->slab = false;
    if (d->weight_layout == QF_LAYOUT_GEMV_SLAB) {
        if (d->path == QF_PATH_GEMM)
            return bad(QF_ERR_BAD_ARG, "QF_LAYOUT_GEMV_SLAB weights are read by the GEMV path only");
        if (d->N % 64 != 0) return bad(QF_ERR_BAD_ARG, "QF_LAYOUT_GEMV_SLAB needs N to be a multiple of 64");
        if (d->M > QF_SLAB_MAX_M)
            return bad(QF_ERR_UNSUPPORTED, "QF_LAYOUT_GEMV_SLAB serves M <= 32; use a tcgen05 layout for larger batches");
        int grid = 1, depth = 1;
        slab_geometry(d->M, d->N, d->K, kSmCount, d->split_k, &grid, &depth);
        p->slab = true;
        p->path = QF_PATH_GEMV;
        p->split_k = grid;
        p->chunks_per_split = depth;
        p->m_tiles = 1;
        p->bn = 8 * ((slab_m_pad(d->M) + 7) / 8);
        p->ws_partial_bytes = slab_workspace_bytes(grid, d->M);
        p->ws_counter_bytes = 0;
        return QF_OK;
    }

    int path = d->path;
    if (path == QF_PATH_AUTO) {
        // M <= 2: the GEMV kernel wins on small matrices (short start-up, 4 blocks per SM); on large ones the tcgen05
        // kernel streams faster (measured at M=1: 42 MB 24.4 vs 17.7 us, 59 MB 33.0 vs 22.0 us, 117 MB 56.5 vs
        // 36.5 us with prepacked weights; 19.8 / 24.7 / 41.7 us with canonical ones; a tie around 32 MB).
        const int64_t wbytes = d->K * d->N / 2;
        const bool big = d->N % 128 == 0 &&
                         wbytes >= (d->weight_layout == QF_LAYOUT_CANONICAL ? (int64_t)40 << 20 : (int64_t)32 << 20);
        path = (d->M <= 2 && !big) ? QF_PATH_GEMV : QF_PATH_GEMM;
    }
    if (path != QF_PATH_GEMV && path != QF_PATH_GEMM) return bad(QF_ERR_BAD_ARG, "unknown path");
    if (d->epilogue != QF_EPI_NONE) {
        // the fused epilogues live in the streaming GEMV kernel (above) and in the tcgen05 kernel
        if (d->path == QF_PATH_GEMV || d->N % 128 != 0)
            return bad(QF_ERR_UNSUPPORTED,
                       "a fused epilogue needs QF_LAYOUT_GEMV_SLAB weights or the tcgen05 path (N % 128 == 0)");
        path = QF_PATH_GEMM;
    }
    if (path == QF_PATH_GEMM && d->N % 128 != 0) {
        if (d->path == QF_PATH_GEMM) return bad(QF_ERR_BAD_ARG, "the GEMM path needs N to be a multiple of 128");
        path = QF_PATH_GEMV;
    }
    if (path == QF_PATH_GEMV && d->weight_layout != QF_LAYOUT_CANONICAL) {
        if (d->N % 128 != 0) return bad(QF_ERR_UNSUPPORTED, "interleaved weights need N to be a multiple of 128");
        path = QF_PATH_GEMM;  // only the tcgen05 kernel reads the interleaved layout
    }
    p->path = path;
    const int chunks = (int)(d->K / 128);
    if (path == QF_PATH_GEMV) {
        p->m_tiles = (int)((d->M + 7) / 8);
        if (p->m_tiles < 1) p->m_tiles = 1;
        p->bn = 8;
        const int64_t col_blocks = (d->N + 63) / 64;
        int split;
        if (d->split_k > 0) {
            split = d->split_k;
        } else {
            const int64_t base = col_blocks * p->m_tiles;
            const int64_t target = (int64_t)kSmCount * 4;
            split = (int)((target + base / 2) / base);
            const int max_split = chunks / 4 > 0 ? chunks / 4 : 1;
            if (split > max_split) split = max_split;
            if (split < 1) split = 1;
        }
        if (split > chunks) split = chunks;
        if (d->split_k == 0 && split > 8 && split <= 10 && chunks % 8 == 0 && chunks / 8 <= 32)
            split = 8;  // an even split that fits one thread-block cluster (on-chip reduction)
        int cps = (chunks + split - 1) / split;
        if (cps > 32) cps = 32;
        split = (chunks + cps - 1) / cps;
        p->split_k = split;
        p->chunks_per_split = cps;
        if (col_blocks * p->m_tiles > kMaxCounters) split = 1, cps = chunks > 32 ? 32 : chunks;
        if (cps * split < chunks) return bad(QF_ERR_UNSUPPORTED, "K too large for this N on the GEMV path");
        p->split_k = split;
        p->chunks_per_split = cps;
        if (split > 1) {
            p->ws_partial_bytes = (size_t)split * p->m_tiles * 8 * d->N * sizeof(float);
            p->ws_counter_bytes = kCounterBytes;
        } else {
            p->ws_partial_bytes = 0;
            p->ws_counter_bytes = 0;
        }
    } else {
        const int bn = d->M <= 16 ? 16 : d->M <= 32 ? 32 : d->M <= 64 ? 64 : d->M <= 128 ? 128 : 256;
        const int bk = gemm_block_k(bn);
        const int kblocks = (int)(d->K / bk);
        p->bn = bn;
        p->m_tiles = (int)((d->M + bn - 1) / bn);
        if (p->m_tiles < 1) p->m_tiles = 1;
        const int64_t tiles = (int64_t)p->m_tiles * (d->N / 128);
        int split;
        if (d->split_k > 0) {
            split = d->split_k;
        } else {
            const int64_t slots = (int64_t)kSmCount * (bn <= 64 ? 2 : 1);  // two narrow CTAs fit one SM
            split = (int)(slots / tiles);
            if (split < 1) split = 1;
            // narrow tiles: at most 8 splits, the size of a portable thread-block cluster; 8 splits summed on chip
            // beat 16 or 32 summed through global memory (measured, 8 tiles, K = 8192: 9.3 -> 6.9 us at M = 16,
            // 17.7 -> 9.6 us at M = 64)
            if (bn <= 64 && split > 8) split = 8;
        }
        if (split > kblocks) split = kblocks;
        int kbps = (kblocks + split - 1) / split;
        const int min_kbps = d->split_k > 0 ? 1 : (kblocks < 4 ? kblocks : 4);
        if (kbps < min_kbps) kbps = min_kbps;
        split = (kblocks + kbps - 1) / kbps;
        if (d->split_k == 0 && split > 2 && kblocks % split != 0) {
            // a slightly smaller split that divides K evenly beats an uneven one: fewer partial tiles to write and
            // sum and no short last split (measured on K = 14336: 8 x 14 k-blocks is 3-7 % faster than 8 x 13 + 8)
            for (int s2 = split - 1; s2 >= split - 2 && s2 >= 2; --s2)
                if (kblocks % s2 == 0 && (kblocks / s2) * 20 <= kbps * 23) {
                    split = s2;
                    kbps = kblocks / s2;
                    break;
                }
        }
        if (d->split_k == 0 && bn <= 64 && split >= 2 && split <= 8 && tiles * split > kClusterMaxBlocks &&
            kClusterMaxBlocks / tiles >= 2) {
            // A launch of more than kClusterMaxBlocks blocks cannot run as one wave of thread-block clusters and
            // would sum its partial tiles through global memory; fewer, longer splits that keep the on-chip
            // reduction are faster (measured, 48 tiles: 6 splits 10.0 / 15.8 us at M = 16 / 64, 5 splits 9.1 / 11.9).
            split = (int)(kClusterMaxBlocks / tiles);
            kbps = (kblocks + split - 1) / split;
            split = (kblocks + kbps - 1) / kbps;
        }
        if (tiles > kMaxCounters) split = 1, kbps = kblocks;
        p->split_k = split;
        p->chunks_per_split = kbps;
        if (split > 1) {
            p->ws_partial_bytes = (size_t)split * p->m_tiles * bn * d->N * sizeof(float);
            p->ws_counter_bytes = kCounterBytes;
        } else {
            p->ws_partial_bytes = 0;
            p->ws_counter_bytes = 0;
        }
    }
    return QF_OK;
}

static int check_linear_args(qf_ctx *ctx, const qf_linear_desc *d, const void *X, const void *qw, const void *scales,
                             const void *zeros, const void *Y) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (d->weight_layout == QF_LAYOUT_GEMV_SLAB) {
        // the blob carries scales and zeros
        if (!X || !qw || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
        if (!aligned16(X) || !aligned16(qw) || !aligned16(Y))
            return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
        return QF_OK;
    }
    if (!X || !qw || !scales || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (d->zero_mode != QF_ZERO_CONST && !zeros) return fail(ctx, QF_ERR_BAD_ARG, "zero_mode needs a qzeros tensor");
    if (d->zero_mode == QF_ZERO_U4 && d->N % 8 != 0) return fail(ctx, QF_ERR_BAD_ARG, "QF_ZERO_U4 needs N % 8 == 0");
    if (!aligned16(X) || !aligned16(qw) || !aligned16(scales) || !aligned16(Y) || (zeros && !aligned16(zeros)))
        return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    return QF_OK;
}

}  // namespace qf

using namespace qf;

extern "C" {

int qf_version(void) { return QF_RT_VERSION; }

const char *qf_status_string(int status) {
    switch (status) {
        case QF_OK: return "QF_OK";
        case QF_ERR_BAD_ARG: return "QF_ERR_BAD_ARG";
        case QF_ERR_UNSUPPORTED: return "QF_ERR_UNSUPPORTED";
        case QF_ERR_CUDA: return "QF_ERR_CUDA";
        case QF_ERR_NCCL: return "QF_ERR_NCCL";
        case QF_ERR_TIMEOUT: return "QF_ERR_TIMEOUT";
        case QF_ERR_UNIMPLEMENTED: return "QF_ERR_UNIMPLEMENTED";
        case QF_ERR_WORKSPACE: return "QF_ERR_WORKSPACE";
        default: return "QF_ERR_UNKNOWN";
    }
}

int qf_ctx_create(qf_ctx **out, int device) {
    if (!out) return QF_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return QF_ERR_CUDA;  // no CPU fallback exists
    if (device < 0 || device >= count) return QF_ERR_BAD_ARG;
    DeviceGuard guard(device);  // the caller's current device is restored on every return path
    if (!guard.ok()) return QF_ERR_CUDA;
    qf_ctx *ctx = new (std::nothrow) qf_ctx();
    if (!ctx) return QF_ERR_CUDA;
    ctx->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete ctx;
        return QF_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (prop.major != 10) {
        delete ctx;
        return QF_ERR_UNSUPPORTED;  // built for sm_100a only
    }
    int st = gemv_init(ctx);
    if (st == QF_OK) st = gemm_init(ctx);
    if (st == QF_OK) st = gemv_slab_init(ctx);
    if (st != QF_OK) {
        delete ctx;
        return st;
    }
    *out = ctx;
    return QF_OK;
}

int qf_ctx_destroy(qf_ctx *ctx) {
    if (!ctx) return QF_OK;
    DeviceGuard guard(ctx->device);
    cudaDeviceSynchronize();
    for (auto &sl : ctx->host_slot) {
        if (sl.x) cudaFree(sl.x);
        if (sl.y) cudaFree(sl.y);
        if (sl.copied_in) cudaEventDestroy(sl.copied_in);
        if (sl.kernel_done) cudaEventDestroy(sl.kernel_done);
    }
    for (void *q : ctx->retired) cudaFree(q);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    delete ctx;
    return QF_OK;
}

const char *qf_last_error(const qf_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int qf_unpack_int4(qf_ctx *ctx, const void *packed_i8, void *out_i8, int64_t rows, int64_t packed_cols, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (rows < 0 || packed_cols < 0) return fail(ctx, QF_ERR_BAD_ARG, "negative extent");
    if (rows == 0 || packed_cols == 0) return QF_OK;
    if (!packed_i8 || !out_i8) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (((uintptr_t)out_i8 & 1u) != 0) return fail(ctx, QF_ERR_BAD_ARG, "output must be 2-byte aligned");
    return launch_unpack(ctx, packed_i8, out_i8, rows, packed_cols, (cudaStream_t)stream);
}

int qf_dequant_w4(qf_ctx *ctx, const qf_linear_desc *desc, const void *qweight, const void *scales,
                  const void *qzeros_or_null, void *w_out, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (!desc) return fail(ctx, QF_ERR_BAD_ARG, "desc is null");
    if (desc->weight_layout != QF_LAYOUT_CANONICAL)
        return fail(ctx, QF_ERR_UNSUPPORTED, "qf_dequant_w4 reads canonical weights only (undo the prepack first)");
    qf_linear_desc d = *desc;
    d.M = 1;
    d.path = QF_PATH_GEMV;
    d.out_dtype = d.act_dtype;
    d.epilogue = QF_EPI_NONE;
    Plan plan;
    std::string why;
    int st = make_plan(&d, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    st = check_linear_args(ctx, &d, w_out, qweight, scales, qzeros_or_null, w_out);
    if (st != QF_OK) return st;
    return launch_dequant(ctx, &d, qweight, scales, qzeros_or_null, w_out, (cudaStream_t)stream);
}

size_t qf_w4a16_workspace_bytes(const qf_linear_desc *desc) {
    Plan plan;
    if (make_plan(desc, &plan, nullptr) != QF_OK) return 0;
    return plan.ws_partial_bytes + plan.ws_counter_bytes;
}

int qf_w4a16_plan(const qf_linear_desc *desc, int32_t *path_out, int32_t *split_k_out) {
    Plan plan;
    int st = make_plan(desc, &plan, nullptr);
    if (st != QF_OK) return st;
    if (path_out) *path_out = plan.path;
    if (split_k_out) *split_k_out = plan.split_k;
    return QF_OK;
}

int qf_w4a16_linear_fused(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight,
                          const void *scales, const void *qzeros_or_null, void *Y, const void *residual,
                          void *workspace, size_t workspace_bytes, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    Plan plan;
    std::string why;
    int st = make_plan(desc, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    if (desc->M == 0) return QF_OK;
    st = check_linear_args(ctx, desc, X, qweight, scales, qzeros_or_null, Y);
    if (st != QF_OK) return st;
    st = check_current_device(ctx);
    if (st != QF_OK) return st;
    if (desc->epilogue == QF_EPI_RESIDUAL_ADD && (!residual || !aligned16(residual)))
        return fail(ctx, QF_ERR_BAD_ARG, "QF_EPI_RESIDUAL_ADD needs a 16-byte aligned residual tensor");
    if (desc->epilogue == QF_EPI_SILU_MUL && desc->N % 16 != 0)
        return fail(ctx, QF_ERR_BAD_ARG, "QF_EPI_SILU_MUL needs N (gate and up rows together) to be a multiple of 16");
    const size_t need = plan.ws_partial_bytes + plan.ws_counter_bytes;
    if (need > 0) {
        if (!workspace || workspace_bytes < need)
            return fail(ctx, QF_ERR_WORKSPACE, "workspace smaller than qf_w4a16_workspace_bytes(desc)");
        if (!aligned16(workspace)) return fail(ctx, QF_ERR_BAD_ARG, "workspace must be 16-byte aligned");
    }
    if (plan.slab)
        return launch_gemv_slab(ctx, desc, plan, X, qweight, Y, residual, workspace, (cudaStream_t)stream);
    if (plan.path == QF_PATH_GEMV)
        return launch_gemv(ctx, desc, plan, X, qweight, scales, qzeros_or_null, Y, workspace, (cudaStream_t)stream);
    return launch_gemm(ctx, desc, plan, X, qweight, scales, qzeros_or_null, Y, residual, workspace,
                       (cudaStream_t)stream);
}

int qf_w4a16_linear(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight, const void *scales,
                    const void *qzeros_or_null, void *Y, void *workspace, size_t workspace_bytes, void *stream) {
    if (desc && desc->epilogue == QF_EPI_RESIDUAL_ADD)
        return fail(ctx, QF_ERR_BAD_ARG, "QF_EPI_RESIDUAL_ADD takes its residual through qf_w4a16_linear_fused");
    return qf_w4a16_linear_fused(ctx, desc, X, qweight, scales, qzeros_or_null, Y, nullptr, workspace, workspace_bytes,
                                 stream);
}

int qf_w4a16_linear_batched(qf_ctx *ctx, int count, const qf_linear_desc *descs, const void *const *X,
                            const void *const *qweight, const void *const *scales, const void *const *qzeros,
                            void *const *Y, const void *const *residual, void *workspace, size_t workspace_bytes,
                            void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (count < 0) return fail(ctx, QF_ERR_BAD_ARG, "negative count");
    if (count == 0) return QF_OK;
    if (!descs || !X || !qweight || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null argument array");
    for (int i = 0; i < count; ++i) {
        const int st = qf_w4a16_linear_fused(ctx, &descs[i], X[i], qweight[i], scales ? scales[i] : nullptr,
                                             qzeros ? qzeros[i] : nullptr, Y[i], residual ? residual[i] : nullptr,
                                             workspace, workspace_bytes, stream);
        if (st != QF_OK) {
            ctx->last_error = "entry " + std::to_string(i) + ": " + ctx->last_error;
            return st;
        }
    }
    return QF_OK;
}

size_t qf_prepack_bytes(int layout, int64_t N, int64_t K) {
    if (N <= 0 || K <= 0 || K % 128 != 0) return 0;
    switch (layout) {
        case QF_LAYOUT_CANONICAL: return (size_t)N * (size_t)K / 2;
        case QF_LAYOUT_INTERLEAVED:
        case QF_LAYOUT_TILED: return N % 128 == 0 ? (size_t)N * (size_t)K / 2 : 0;
        case QF_LAYOUT_GEMV_SLAB: return N % 64 == 0 ? (size_t)(N / 64) * (size_t)(K / 128) * QF_SLAB_UNIT_BYTES : 0;
        default: return 0;
    }
}

int qf_prepack_gemv_slab(qf_ctx *ctx, const qf_linear_desc *desc, const void *qweight, const void *scales,
                         const void *qzeros_or_null, void *blob_out, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (!desc) return fail(ctx, QF_ERR_BAD_ARG, "desc is null");
    qf_linear_desc d = *desc;
    d.M = 1;
    d.path = QF_PATH_AUTO;
    d.weight_layout = QF_LAYOUT_GEMV_SLAB;
    d.epilogue = QF_EPI_NONE;
    d.out_dtype = d.act_dtype;
    Plan plan;
    std::string why;
    int st = make_plan(&d, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    if (!qweight || !scales || !blob_out) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (d.zero_mode != QF_ZERO_CONST && !qzeros_or_null) return fail(ctx, QF_ERR_BAD_ARG, "zero_mode needs a qzeros tensor");
    if (!aligned16(qweight) || !aligned16(scales) || !aligned16(blob_out) || (qzeros_or_null && !aligned16(qzeros_or_null)))
        return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    if (blob_out == qweight) return fail(ctx, QF_ERR_BAD_ARG, "the blob must not alias the canonical weights");
    st = check_current_device(ctx);
    if (st != QF_OK) return st;
    return launch_slab_prepack(ctx, &d, qweight, scales, qzeros_or_null, blob_out, (cudaStream_t)stream);
}

int qf_unpack_gemv_slab(qf_ctx *ctx, int64_t N, int64_t K, const void *blob, void *qweight_out, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (N <= 0 || K <= 0 || N % 64 != 0 || K % 128 != 0)
        return fail(ctx, QF_ERR_BAD_ARG, "QF_LAYOUT_GEMV_SLAB needs N % 64 == 0 and K % 128 == 0");
    if (!blob || !qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (!aligned16(blob) || !aligned16(qweight_out)) return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    int st = check_current_device(ctx);
    if (st != QF_OK) return st;
    return launch_slab_unpack(ctx, N, K, blob, qweight_out, (cudaStream_t)stream);
}

int qf_repack_kn_to_canonical(qf_ctx *ctx, const void *w_kn, int packed_along_n, int64_t K, int64_t N,
                              void *qweight_out, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (K <= 0 || N <= 0 || K % 8 != 0 || N % 2 != 0)
        return fail(ctx, QF_ERR_BAD_ARG, "qf_repack_kn_to_canonical needs K % 8 == 0 and N % 2 == 0");
    if (!w_kn || !qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (w_kn == qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "in and out must not alias");
    if (((uintptr_t)qweight_out & 3u) != 0) return fail(ctx, QF_ERR_BAD_ARG, "output must be 4-byte aligned");
    int st = check_current_device(ctx);
    if (st != QF_OK) return st;
    return launch_repack_kn(ctx, w_kn, packed_along_n ? 1 : 0, K, N, qweight_out, (cudaStream_t)stream);
}

int qf_w4a16_gemv_static_scratch(qf_ctx *ctx, const qf_linear_desc *desc, const void *X, const void *qweight,
                                 const void *scales, const void *qzeros_or_null, void *Y, void *stream) {
    if (!desc) return fail(ctx, QF_ERR_BAD_ARG, "desc is null");
    qf_linear_desc d = *desc;
    d.path = QF_PATH_GEMV;
    if (d.weight_layout != QF_LAYOUT_CANONICAL)
        return fail(ctx, QF_ERR_UNSUPPORTED, "the GEMV kernel reads canonical weights only");
    Plan plan;
    std::string why;
    int st = make_plan(&d, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    if (d.M == 0) return QF_OK;
    if (!X || !qweight || !scales || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (d.zero_mode != QF_ZERO_CONST && !qzeros_or_null) return fail(ctx, QF_ERR_BAD_ARG, "zero_mode needs a qzeros tensor");
    if (!aligned16(X) || !aligned16(qweight) || !aligned16(scales) || !aligned16(Y) ||
        (qzeros_or_null && !aligned16(qzeros_or_null)))
        return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    return launch_gemv_static(ctx, &d, plan, X, qweight, scales, qzeros_or_null, Y, (cudaStream_t)stream);
}

// Staging buffers only grow; the outgrown one is retired, not freed (see qf_ctx::HostSlot).
static int grow(qf_ctx *ctx, void **buf, size_t *have, size_t need) {
    if (*have >= need) return QF_OK;
    if (*buf) ctx->retired.push_back(*buf);
    *buf = nullptr;
    *have = 0;
    size_t cap = (need + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    QF_CUDA_TRY(ctx, cudaMalloc(buf, cap));
    *have = cap;
    return QF_OK;
}

int qf_w4a16_linear_host_async(qf_ctx *ctx, const qf_linear_desc *desc, const void *X_host, const void *qweight,
                         const void *scales, const void *qzeros_or_null, void *Y_host, void *workspace,
                         size_t workspace_bytes, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (!desc) return fail(ctx, QF_ERR_BAD_ARG, "desc is null");
    if (!X_host || !Y_host) return fail(ctx, QF_ERR_BAD_ARG, "null host pointer");
    if (desc->M == 0) return QF_OK;
    if (desc->M < 0 || desc->N <= 0 || desc->K <= 0) return fail(ctx, QF_ERR_BAD_ARG, "bad shape");
    int st = check_current_device(ctx);
    if (st != QF_OK) return st;
    const size_t xb = (size_t)desc->M * desc->K * 2;
    const int64_t out_cols = desc->epilogue == QF_EPI_SILU_MUL ? desc->N / 2 : desc->N;
    const size_t yb = (size_t)desc->M * out_cols * (desc->out_dtype == QF_F32 ? 4 : 2);
    if (!ctx->copy_stream) {
        QF_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
        for (auto &sl : ctx->host_slot) {
            QF_CUDA_TRY(ctx, cudaEventCreateWithFlags(&sl.copied_in, cudaEventDisableTiming));
            QF_CUDA_TRY(ctx, cudaEventCreateWithFlags(&sl.kernel_done, cudaEventDisableTiming));
        }
    }
    qf_ctx::HostSlot &sl = ctx->host_slot[ctx->host_next];
    ctx->host_next ^= 1;
    st = grow(ctx, &sl.x, &sl.x_bytes, xb);
    if (st != QF_OK) return st;
    st = grow(ctx, &sl.y, &sl.y_bytes, yb);
    if (st != QF_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;
    // activations: on the copy stream, as soon as the slot's previous kernel (two calls ago) has read its own
    QF_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream, sl.kernel_done, 0));  // no-op before the first record
    QF_CUDA_TRY(ctx, cudaMemcpyAsync(sl.x, X_host, xb, cudaMemcpyHostToDevice, ctx->copy_stream));
    QF_CUDA_TRY(ctx, cudaEventRecord(sl.copied_in, ctx->copy_stream));
    QF_CUDA_TRY(ctx, cudaStreamWaitEvent(s, sl.copied_in, 0));
    st = qf_w4a16_linear(ctx, desc, sl.x, qweight, scales, qzeros_or_null, sl.y, workspace, workspace_bytes, stream);
    if (st != QF_OK) return st;
    QF_CUDA_TRY(ctx, cudaEventRecord(sl.kernel_done, s));
    // the result goes back on the caller's stream: synchronising it is all the caller has to do
    QF_CUDA_TRY(ctx, cudaMemcpyAsync(Y_host, sl.y, yb, cudaMemcpyDeviceToHost, s));
    return QF_OK;
}

int qf_w4a16_linear_host(qf_ctx *ctx, const qf_linear_desc *desc, const void *X_host, const void *qweight,
                         const void *scales, const void *qzeros_or_null, void *Y_host, void *workspace,
                         size_t workspace_bytes, void *stream) {
    const int st = qf_w4a16_linear_host_async(ctx, desc, X_host, qweight, scales, qzeros_or_null, Y_host, workspace,
                                              workspace_bytes, stream);
    if (st != QF_OK) return st;
    QF_CUDA_TRY(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return QF_OK;
}

int qf_prepack_w4(qf_ctx *ctx, const void *qweight_in, void *qweight_out, int64_t n_words, int to_canonical,
                  void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (n_words < 0) return fail(ctx, QF_ERR_BAD_ARG, "negative extent");
    if (n_words == 0) return QF_OK;
    if (!qweight_in || !qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (((uintptr_t)qweight_in & 3u) || ((uintptr_t)qweight_out & 3u))
        return fail(ctx, QF_ERR_BAD_ARG, "weights must be 4-byte aligned");
    return launch_prepack(ctx, qweight_in, qweight_out, n_words, to_canonical, (cudaStream_t)stream);
}

int qf_prepack_w4_tiled(qf_ctx *ctx, const void *qweight_in, void *qweight_out, int64_t N, int64_t K,
                        int to_canonical, void *stream) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (N <= 0 || K <= 0 || N % 128 != 0 || K % 128 != 0)
        return fail(ctx, QF_ERR_BAD_ARG, "the tiled layout needs N and K to be multiples of 128");
    if (!qweight_in || !qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (qweight_in == qweight_out) return fail(ctx, QF_ERR_BAD_ARG, "in and out must not alias");
    if (((uintptr_t)qweight_in & 15u) || ((uintptr_t)qweight_out & 15u))
        return fail(ctx, QF_ERR_BAD_ARG, "weights must be 16-byte aligned");
    return launch_prepack_tiled(ctx, qweight_in, qweight_out, N, K, to_canonical, (cudaStream_t)stream);
}

int qf_ctx_status(const qf_ctx *ctx) {
    if (!ctx) return QF_ERR_BAD_ARG;
    return ctx->host_status ? *(volatile int *)ctx->host_status : QF_OK;
}

int qf_ctx_clear_status(qf_ctx *ctx) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (ctx->host_status) *(volatile int *)ctx->host_status = QF_OK;
    return QF_OK;
}

int64_t qf_launch_count(void) { return (int64_t)g_launch_count.load(); }

}  // extern "C"
