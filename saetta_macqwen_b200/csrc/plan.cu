// Record once, replay per token: the reference's Plan / Built on CUDA graphs.
//
// Stands in for src/plan.rs:52-260.  There a Plan is a list of dispatches encoded once
// into an indirect command buffer; what changes between replays is the 16-byte
// TokenParams buffer the kernels read.  Here the recording is a stream capture: between
// begin and build the caller issues this library's entry points (or its own kernels)
// on the plan's stream, passing the plan's TokenParams pointer wherever an entry point
// takes one; build turns the capture into an executable graph.  set_params writes the
// host copy of TokenParams; the graph's first node copies it to the device, so a replay
// is one graph launch.  `op` is stream order; `op_parallel` is a side stream forked from
// and joined back into the plan's stream (saetta_plan_parallel_begin / _end).
#include <new>

#include "host.hpp"

using namespace saetta;

struct saetta_plan {
    int device = 0;
    cudaStream_t stream = nullptr, side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr, t0 = nullptr, t1 = nullptr;
    saetta_token_params *params_dev = nullptr;
    saetta_token_params *params_host = nullptr; // pinned
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    bool recording = false, side_open = false;
};

extern "C" {

int saetta_plan_create(int device, saetta_plan **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "Plan::new: out is null");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "Plan::new: cannot select the device");
    auto *p = new (std::nothrow) saetta_plan();
    if (!p) return fail(SAETTA_ERR_NO_MEM, "Plan::new: host allocation");
    p->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&p->t0);
    if (e == cudaSuccess) e = cudaEventCreate(&p->t1);
    if (e == cudaSuccess) e = cudaMalloc((void **)&p->params_dev, sizeof(saetta_token_params));
    if (e == cudaSuccess) e = cudaMemset(p->params_dev, 0, sizeof(saetta_token_params));
    if (e == cudaSuccess) e = cudaMallocHost((void **)&p->params_host, sizeof(saetta_token_params));
    if (e != cudaSuccess) {
        saetta_plan_destroy(p);
        return cuda_fail(e, "Plan::new");
    }
    *p->params_host = saetta_token_params{0, 0, 1, 0};
    *out = p;
    return SAETTA_OK;
}

void saetta_plan_destroy(saetta_plan *p) {
    if (!p) return;
    DeviceGuard guard(p->device);
    if (p->recording) { // an abandoned recording: end the capture so the stream can be destroyed
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(p->stream, &g);
        if (g) cudaGraphDestroy(g);
    }
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    if (p->stream) cudaStreamDestroy(p->stream);
    if (p->side) cudaStreamDestroy(p->side);
    for (cudaEvent_t ev : {p->fork, p->join, p->t0, p->t1})
        if (ev) cudaEventDestroy(ev);
    cudaFree(p->params_dev);
    cudaFreeHost(p->params_host);
    delete p;
}

const saetta_token_params *saetta_plan_params(const saetta_plan *p) { return p ? p->params_dev : nullptr; }
void *saetta_plan_stream(const saetta_plan *p) { return p ? (void *)p->stream : nullptr; }

int saetta_plan_begin(saetta_plan *p) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Plan: null pointer");
    if (p->recording) return fail(SAETTA_ERR_BAD_ARG, "Plan: already recording");
    DeviceGuard guard(p->device);
    if (p->exec) cudaGraphExecDestroy(p->exec), p->exec = nullptr;
    if (p->graph) cudaGraphDestroy(p->graph), p->graph = nullptr;
    SAETTA_CUDA(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal));
    p->recording = true;
    // first node of every replay: the per-token values, from the pinned host copy
    cudaError_t e = cudaMemcpyAsync(p->params_dev, p->params_host, sizeof(saetta_token_params), cudaMemcpyHostToDevice, p->stream);
    if (e != cudaSuccess) return cuda_fail(e, "Plan: recording the TokenParams upload");
    return SAETTA_OK;
}

int saetta_plan_parallel_begin(saetta_plan *p, void **side_stream) {
    if (!p || !side_stream) return fail(SAETTA_ERR_BAD_ARG, "Plan::op_parallel: null pointer");
    if (!p->recording || p->side_open) return fail(SAETTA_ERR_BAD_ARG, "Plan::op_parallel: not recording, or a side branch is already open");
    DeviceGuard guard(p->device);
    SAETTA_CUDA(cudaEventRecord(p->fork, p->stream));
    SAETTA_CUDA(cudaStreamWaitEvent(p->side, p->fork, 0));
    p->side_open = true;
    *side_stream = p->side;
    return SAETTA_OK;
}

int saetta_plan_parallel_end(saetta_plan *p) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Plan: null pointer");
    if (!p->side_open) return fail(SAETTA_ERR_BAD_ARG, "Plan::op_parallel: no side branch is open");
    DeviceGuard guard(p->device);
    SAETTA_CUDA(cudaEventRecord(p->join, p->side));
    SAETTA_CUDA(cudaStreamWaitEvent(p->stream, p->join, 0));
    p->side_open = false;
    return SAETTA_OK;
}

int saetta_plan_build(saetta_plan *p) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Plan: null pointer");
    if (!p->recording) return fail(SAETTA_ERR_BAD_ARG, "Plan::build: nothing is being recorded");
    DeviceGuard guard(p->device);
    if (p->side_open)
        if (int rc = saetta_plan_parallel_end(p)) return rc;
    p->recording = false;
    SAETTA_CUDA(cudaStreamEndCapture(p->stream, &p->graph));
    SAETTA_CUDA(cudaGraphInstantiate(&p->exec, p->graph, 0));
    return SAETTA_OK;
}

int saetta_plan_len(const saetta_plan *p, size_t *ops) {
    if (!p || !ops) return fail(SAETTA_ERR_BAD_ARG, "Plan::len: null pointer");
    if (!p->graph) return fail(SAETTA_ERR_BAD_ARG, "Plan::len: the plan has not been built");
    size_t n = 0;
    SAETTA_CUDA(cudaGraphGetNodes(p->graph, nullptr, &n));
    std::vector<cudaGraphNode_t> nodes(n);
    if (n) SAETTA_CUDA(cudaGraphGetNodes(p->graph, nodes.data(), &n));
    size_t kernels = 0;
    for (cudaGraphNode_t node : nodes) {
        cudaGraphNodeType t;
        SAETTA_CUDA(cudaGraphNodeGetType(node, &t));
        kernels += t == cudaGraphNodeTypeKernel;
    }
    *ops = kernels;
    return SAETTA_OK;
}

int saetta_plan_set_params(saetta_plan *p, uint32_t token, uint32_t position) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Plan::set_params: null pointer");
    *p->params_host = saetta_token_params{token, position, position + 1, 0};
    return SAETTA_OK;
}

int saetta_plan_commit(saetta_plan *p) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Built::commit: null pointer");
    if (!p->exec) return fail(SAETTA_ERR_BAD_ARG, "Built::commit: the plan has not been built");
    DeviceGuard guard(p->device);
    SAETTA_CUDA(cudaEventRecord(p->t0, p->stream));
    SAETTA_CUDA(cudaGraphLaunch(p->exec, p->stream));
    SAETTA_CUDA(cudaEventRecord(p->t1, p->stream));
    return SAETTA_OK;
}

int saetta_plan_wait(saetta_plan *p) {
    if (!p) return fail(SAETTA_ERR_BAD_ARG, "Pending::wait: null pointer");
    DeviceGuard guard(p->device);
    SAETTA_CUDA(cudaStreamSynchronize(p->stream));
    return SAETTA_OK;
}

int saetta_plan_run(saetta_plan *p) {
    if (int rc = saetta_plan_commit(p)) return rc;
    return saetta_plan_wait(p);
}

int saetta_plan_run_timed(saetta_plan *p, float *gpu_ms) {
    if (!gpu_ms) return fail(SAETTA_ERR_BAD_ARG, "Built::run_timed: null pointer");
    if (int rc = saetta_plan_run(p)) return rc;
    DeviceGuard guard(p->device);
    SAETTA_CUDA(cudaEventElapsedTime(gpu_ms, p->t0, p->t1));
    return SAETTA_OK;
}

} // extern "C"
