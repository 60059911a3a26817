// Exchange buffers for row-parallel linears: one buffer per GPU, every rank maps every other rank's buffer
// (CUDA IPC within one node, NVLink peer access), and the GEMV kernel sums the partial outputs across GPUs
// in its own epilogue (qf_gemv.cu, AR instantiations). Nothing here runs in the hot call except building
// the kernel's pointer table from the already mapped buffers.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "qf_common.cuh"

struct qf_comm {
    qf_ctx *ctx = nullptr;
    int rank = 0;
    int world = 1;
    size_t slot_elems = 0;
    size_t bytes = 0;
    void *local = nullptr;
    void *peer[qf::kMaxPeers] = {nullptr};
    bool peer_is_ipc[qf::kMaxPeers] = {false};  // mapped with cudaIpcOpenMemHandle (to be closed), not a same-process buffer
    bool connected = false;
    long long wait_cycles = 0;
    cudaIpcMemHandle_t handle;
};

namespace qf {

// Exchange buffers created by THIS process, by handle: an IPC handle cannot be opened in the process that made it,
// so a process that drives several ranks (one thread per GPU, or a test that plays two ranks) gets the pointer from
// here, with peer access enabled when the buffer lives on another GPU.
struct LocalBuffer {
    cudaIpcMemHandle_t handle;
    void *ptr;
    int device;
};
static std::mutex g_local_mutex;
static std::vector<LocalBuffer> g_local_buffers;

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
    ar.wait_cycles = c->wait_cycles;
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
    DeviceGuard guard(ctx->device);
    if (!guard.ok()) return fail(ctx, QF_ERR_CUDA, "cannot make the context's device current");
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
    // How long a collect waits for its peers. QF_EXCHANGE_WAIT_MS shortens it (tests of the time-out path); the
    // conversion assumes the 1.9 GHz the SM clock counter runs at under load.
    c->wait_cycles = kExchangeWaitCycles;
    if (const char *e = std::getenv("QF_EXCHANGE_WAIT_MS")) {
        const long long ms = std::atoll(e);
        if (ms > 0) c->wait_cycles = ms * 1900000LL;
    }
    if (world > 1) {
        std::lock_guard<std::mutex> g(g_local_mutex);
        g_local_buffers.push_back(LocalBuffer{c->handle, c->local, ctx->device});
    }
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
    DeviceGuard guard(ctx->device);
    if (!guard.ok()) return fail(ctx, QF_ERR_CUDA, "cannot make the context's device current");
    for (int r = 0; r < comm->world; ++r) {
        if (r == comm->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * QF_COMM_HANDLE_BYTES, QF_COMM_HANDLE_BYTES);
        void *ptr = nullptr;
        int owner_device = -1;
        {
            std::lock_guard<std::mutex> g(g_local_mutex);
            for (const LocalBuffer &lb : g_local_buffers)
                if (memcmp(&lb.handle, &h, sizeof(h)) == 0) {
                    ptr = lb.ptr;
                    owner_device = lb.device;
                }
        }
        if (ptr) {
            // a buffer of this very process
            if (owner_device != ctx->device) {
                const cudaError_t pe = cudaDeviceEnablePeerAccess(owner_device, 0);
                if (pe == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (pe != cudaSuccess) return cuda_fail(ctx, pe, "qf_comm_connect: cudaDeviceEnablePeerAccess");
            }
        } else {
            cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "qf_comm_connect: cudaIpcOpenMemHandle");
            comm->peer_is_ipc[r] = true;
        }
        comm->peer[r] = ptr;
    }
    comm->connected = true;
    return QF_OK;
}

int qf_comm_destroy(qf_comm *comm) {
    if (!comm) return QF_OK;
    DeviceGuard guard(comm->ctx->device);
    for (int r = 0; r < comm->world; ++r)
        if (r != comm->rank && comm->peer[r] && comm->peer_is_ipc[r]) cudaIpcCloseMemHandle(comm->peer[r]);
    {
        std::lock_guard<std::mutex> g(g_local_mutex);
        for (size_t i = 0; i < g_local_buffers.size(); ++i)
            if (g_local_buffers[i].ptr == comm->local) {
                g_local_buffers.erase(g_local_buffers.begin() + (long)i);
                break;
            }
    }
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
    if (desc->epilogue != QF_EPI_NONE)
        return fail(ctx, QF_ERR_UNSUPPORTED, "the exchanging linears take no fused epilogue");
    qf_linear_desc local_desc = *desc;
    if (local_desc.weight_layout == QF_LAYOUT_GEMV_SLAB && local_desc.split_k == 0) {
        // A collecting thread block waits for its peers while it holds its SM slot, so every thread block of the
        // launch must be resident at once on every rank: an explicit grid of whole multiples of the SM count (the
        // launch checks it against the occupancy the kernel really gets). Same size rule as the plain kernel.
        const long long wbytes = (long long)(local_desc.N / 64) * (local_desc.K / 128) * QF_SLAB_UNIT_BYTES;
        const int per_sm = (wbytes <= kSlabSmallBytes) ? 2 : (local_desc.M > 16 ? 3 : 4);
        local_desc.split_k = per_sm * ctx->sm_count;
        desc = &local_desc;
    }
    Plan plan;
    std::string why;
    int st = make_plan(desc, &plan, &why);
    if (st != QF_OK) return fail(ctx, st, why);
    if (desc->M == 0) return QF_OK;
    st = check_current_device(ctx);
    if (st != QF_OK) return st;
    const bool slab = desc->weight_layout == QF_LAYOUT_GEMV_SLAB;
    if (!X || !qweight || (!slab && !scales) || !Y) return fail(ctx, QF_ERR_BAD_ARG, "null tensor pointer");
    if (!slab && desc->zero_mode != QF_ZERO_CONST && !qzeros_or_null)
        return fail(ctx, QF_ERR_BAD_ARG, "zero_mode needs a qzeros tensor");
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15u) == 0; };
    if (!al16(X) || !al16(qweight) || !al16(Y) ||
        (!slab && (!al16(scales) || (qzeros_or_null && !al16(qzeros_or_null)))))
        return fail(ctx, QF_ERR_BAD_ARG, "device pointers must be 16-byte aligned");
    if (slab && desc->split_k > 0 && desc->split_k > 4 * ctx->sm_count)
        return fail(ctx, QF_ERR_UNSUPPORTED,
                    "an exchanging launch must be resident at once: at most 4 thread blocks per SM");
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
    if (plan.slab)
        return launch_gemv_slab_ar(ctx, desc, plan, X, qweight, Y, workspace, (cudaStream_t)stream, ar);
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
