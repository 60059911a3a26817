// Exchange buffers for row-parallel linears: one buffer per GPU, every rank maps every other rank's buffer
// (CUDA IPC within one node, NVLink peer access), and the GEMV kernel sums the partial outputs across GPUs
// in its own epilogue (qf_gemv.cu, AR instantiations). Nothing here runs in the hot call except building
// the kernel's pointer table from the already mapped buffers.
#include <cstring>

#include "qf_common.cuh"

struct qf_comm {
    qf_ctx *ctx = nullptr;
    int rank = 0;
    int world = 1;
    size_t slot_elems = 0;
    size_t bytes = 0;
    void *local = nullptr;
    void *peer[qf::kMaxPeers] = {nullptr};
    bool connected = false;
    cudaIpcMemHandle_t handle;
};

namespace qf {

static ArParams comm_params(const qf_comm *c) {
    ArParams ar = {};
    for (int r = 0; r < c->world; ++r) ar.slots[r] = (uint2 *)((char *)c->peer[r] + kCommHeaderBytes);
    ar.local_slots = ar.slots[c->rank];
    ar.epoch = (unsigned *)c->local;
    ar.done = (unsigned *)c->local + 1;
    ar.status = c->ctx->dev_status;
    ar.slot_elems = c->slot_elems;
    ar.world = c->world;
    ar.rank = c->rank;
    return ar;
}

}  // namespace qf

using namespace qf;

extern "C" {

int qf_comm_create(qf_ctx *ctx, int rank, int world, size_t max_out_elems, qf_comm **out) {
    if (!ctx || !out) return QF_ERR_BAD_ARG;
    *out = nullptr;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(ctx, QF_ERR_BAD_ARG, "qf_comm_create: need 1 <= world <= 8 and 0 <= rank < world");
    if (max_out_elems == 0) return fail(ctx, QF_ERR_BAD_ARG, "qf_comm_create: max_out_elems must be positive");
    if (!ctx->dev_status) return fail(ctx, QF_ERR_CUDA, "context has no device status word");
    QF_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    qf_comm *c = new (std::nothrow) qf_comm();
    if (!c) return fail(ctx, QF_ERR_CUDA, "out of host memory");
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    c->slot_elems = (max_out_elems + 63) & ~(size_t)63;
    c->bytes = kCommHeaderBytes + (size_t)2 * world * c->slot_elems * sizeof(uint2);
    cudaError_t e = cudaMalloc(&c->local, c->bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&c->handle, c->local);
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        delete c;
        return cuda_fail(ctx, e, "qf_comm_create");
    }
    c->peer[rank] = c->local;
    c->connected = (world == 1);
    *out = c;
    return QF_OK;
}

int qf_comm_export(const qf_comm *comm, void *handle_out) {
    if (!comm || !handle_out) return QF_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == QF_COMM_HANDLE_BYTES, "handle size");
    if (comm->world == 1) {
        memset(handle_out, 0, QF_COMM_HANDLE_BYTES);
    } else {
        memcpy(handle_out, &comm->handle, QF_COMM_HANDLE_BYTES);
    }
    return QF_OK;
}

int qf_comm_connect(qf_comm *comm, const void *handles, int n_handles) {
    if (!comm) return QF_ERR_BAD_ARG;
    qf_ctx *ctx = comm->ctx;
    if (comm->connected) return QF_OK;
    if (!handles || n_handles != comm->world)
        return fail(ctx, QF_ERR_BAD_ARG, "qf_comm_connect: one handle per rank, in rank order");
    QF_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    for (int r = 0; r < comm->world; ++r) {
        if (r == comm->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * QF_COMM_HANDLE_BYTES, QF_COMM_HANDLE_BYTES);
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qf_comm_connect: cudaIpcOpenMemHandle");
        comm->peer[r] = ptr;
    }
    comm->connected = true;
    return QF_OK;
}

int qf_comm_destroy(qf_comm *comm) {
    if (!comm) return QF_OK;
    cudaSetDevice(comm->ctx->device);
    for (int r = 0; r < comm->world; ++r)
        if (r != comm->rank && comm->peer[r]) cudaIpcCloseMemHandle(comm->peer[r]);
    if (comm->local) cudaFree(comm->local);
    delete comm;
    return QF_OK;
}

// Shared body of the two exchange entry points. The path follows the plan of qf_w4a16_linear (GEMV kernel for
// M <= 2 or when N is not a multiple of 128, tcgen05 kernel otherwise) unless desc->path names one.
static int linear_exchange(qf_ctx *ctx, qf_comm *comm, const qf_linear_desc *desc, const void *X,
                           const void *qweight, const void *scales, const void *qzeros_or_null, void *Y,
                           void *workspace, size_t workspace_bytes, void *stream, int gather) {
    if (!ctx) return QF_ERR_BAD_ARG;
    if (!comm || comm->ctx != ctx) return fail(ctx, QF_ERR_BAD_ARG, "comm is null or belongs to another context");
    if (!comm->connected) return fail(ctx, QF_ERR_BAD_ARG, "qf_comm_connect has not been called");
    if (!desc) return fail(ctx, QF_ERR_BAD_ARG, "desc is null");
    if (desc->M > 64)
        return fail(ctx, QF_ERR_UNSUPPORTED,
                    "the in-kernel exchange serves M <= 64; larger batches are bandwidth-bound on the links and "
                    "should follow the linear with a bulk collective");
    Plan plan;
    std::string why;
    int st = make_plan(desc, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    if (desc->M == 0) return QF_OK;
    if (!X || !qweight || !scales || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (desc->zero_mode != QF_ZERO_CONST && !qzeros_or_null)
        return fail(ctx, QF_ERR_BAD_ARG, "zero_mode needs a qzeros tensor");
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15u) == 0; };
    if (!al16(X) || !al16(qweight) || !al16(scales) || !al16(Y) || (qzeros_or_null && !al16(qzeros_or_null)))
        return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    if ((size_t)desc->M * (size_t)desc->N > comm->slot_elems)
        return fail(ctx, QF_ERR_WORKSPACE, "M*N exceeds the max_out_elems this comm was created with");
    const size_t need = plan.ws_partial_bytes + plan.ws_counter_bytes;
    if (need > 0) {
        if (!workspace || workspace_bytes < need)
            return fail(ctx, QF_ERR_WORKSPACE, "workspace smaller than qf_w4a16_workspace_bytes(desc)");
        if (!al16(workspace)) return fail(ctx, QF_ERR_BAD_ARG, "workspace must be 16-byte aligned");
    }
    ArParams ar = comm_params(comm);
    ar.gather = gather;
    if (plan.path == QF_PATH_GEMV)
        return launch_gemv_ar(ctx, desc, plan, X, qweight, scales, qzeros_or_null, Y, workspace,
                              (cudaStream_t)stream, ar);
    return launch_gemm_ar(ctx, desc, plan, X, qweight, scales, qzeros_or_null, Y, workspace, (cudaStream_t)stream,
                          ar);
}

int qf_w4a16_linear_allreduce(qf_ctx *ctx, qf_comm *comm, const qf_linear_desc *desc, const void *X,
                              const void *qweight, const void *scales, const void *qzeros_or_null, void *Y,
                              void *workspace, size_t workspace_bytes, void *stream) {
    return linear_exchange(ctx, comm, desc, X, qweight, scales, qzeros_or_null, Y, workspace, workspace_bytes, stream,
                           0);
}

int qf_w4a16_linear_allgather(qf_ctx *ctx, qf_comm *comm, const qf_linear_desc *desc, const void *X,
                              const void *qweight, const void *scales, const void *qzeros_or_null, void *Y,
                              void *workspace, size_t workspace_bytes, void *stream) {
    return linear_exchange(ctx, comm, desc, X, qweight, scales, qzeros_or_null, Y, workspace, workspace_bytes, stream,
                           1);
}

}  // extern "C"
