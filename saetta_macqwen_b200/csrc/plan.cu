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
//
// Plan::build_where (src/plan.rs:190-226) -- a replay of only the ops whose kernel a predicate
// keeps, with or without the barriers between them, which src/profile.rs:39-121 uses to time each
// kernel's ops alone -- is a second graph made from the recorded one: the kernel nodes whose
// function name matches, every copy and memset node (the TokenParams upload among them), and
// either the order of the recording carried over the dropped nodes, or no order at all between the kernels.
#include <algorithm>
#include <cstring>
#include <map>
#include <new>
#include <string>

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
    std::vector<std::string> kernel_names; // of the last build, filled on demand
    std::vector<size_t> kernel_ops;
};

struct saetta_built {
    int device = 0;
    cudaStream_t stream = nullptr; // the plan's (borrowed)
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    size_t kernels = 0;
    std::map<cudaGraphNode_t, bool> is_kernel; // nodes of `graph`
};

namespace {

struct Recorded {
    std::vector<cudaGraphNode_t> order;                       // topological
    std::map<cudaGraphNode_t, std::vector<cudaGraphNode_t>> deps;
};

// The recorded graph's nodes in an order in which every node follows what it depends on.
int recorded_order(cudaGraph_t graph, Recorded &r) {
    size_t n = 0, ne = 0;
    SAETTA_CUDA(cudaGraphGetNodes(graph, nullptr, &n));
    std::vector<cudaGraphNode_t> nodes(n);
    if (n) SAETTA_CUDA(cudaGraphGetNodes(graph, nodes.data(), &n));
    SAETTA_CUDA(cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &ne));
    std::vector<cudaGraphNode_t> from(ne), to(ne);
    std::vector<cudaGraphEdgeData> data(ne);
    if (ne) SAETTA_CUDA(cudaGraphGetEdges_v2(graph, from.data(), to.data(), data.data(), &ne));
    std::map<cudaGraphNode_t, size_t> waiting;
    std::map<cudaGraphNode_t, std::vector<cudaGraphNode_t>> next;
    for (cudaGraphNode_t v : nodes) waiting[v] = 0, r.deps[v];
    for (size_t i = 0; i < ne; i++) waiting[to[i]]++, next[from[i]].push_back(to[i]), r.deps[to[i]].push_back(from[i]);
    std::vector<cudaGraphNode_t> ready;
    for (cudaGraphNode_t v : nodes)
        if (!waiting[v]) ready.push_back(v);
    while (!ready.empty()) {
        cudaGraphNode_t v = ready.back();
        ready.pop_back();
        r.order.push_back(v);
        for (cudaGraphNode_t w : next[v])
            if (!--waiting[w]) ready.push_back(w);
    }
    if (r.order.size() != n) return fail(SAETTA_ERR_CUDA, "Plan: the recorded graph has a cycle");
    return SAETTA_OK;
}

int kernel_name(cudaGraphNode_t node, std::string &name, cudaKernelNodeParams &kp) {
    SAETTA_CUDA(cudaGraphKernelNodeGetParams(node, &kp));
    const char *raw = nullptr;
    if (cudaFuncGetName(&raw, kp.func) != cudaSuccess || !raw) {
        cudaGetLastError();
        raw = "?";
    }
    name = raw;
    return SAETTA_OK;
}

} // namespace

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
    p->kernel_names.clear(), p->kernel_ops.clear();
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

// Plan::kernels (src/plan.rs): the distinct kernels of the recording with the number of ops of each,
// in the order of their first op.  names_out[i] points into storage owned by the plan, valid until
// the next saetta_plan_begin or _destroy.  With names_out NULL only *count is written.
int saetta_plan_kernels(saetta_plan *p, const char **names_out, size_t *ops_out, size_t cap, size_t *count) {
    if (!p || !count) return fail(SAETTA_ERR_BAD_ARG, "Plan::kernels: null pointer");
    if (!p->graph) return fail(SAETTA_ERR_BAD_ARG, "Plan::kernels: the plan has not been built");
    DeviceGuard guard(p->device);
    if (p->kernel_names.empty()) {
        Recorded r;
        if (int rc = recorded_order(p->graph, r)) return rc;
        for (cudaGraphNode_t node : r.order) {
            cudaGraphNodeType t;
            SAETTA_CUDA(cudaGraphNodeGetType(node, &t));
            if (t != cudaGraphNodeTypeKernel) continue;
            std::string name;
            cudaKernelNodeParams kp;
            if (int rc = kernel_name(node, name, kp)) return rc;
            size_t i = 0;
            while (i < p->kernel_names.size() && p->kernel_names[i] != name) i++;
            if (i == p->kernel_names.size()) p->kernel_names.push_back(name), p->kernel_ops.push_back(0);
            p->kernel_ops[i]++;
        }
    }
    *count = p->kernel_names.size();
    for (size_t i = 0; names_out && i < cap && i < *count; i++) {
        names_out[i] = p->kernel_names[i].c_str();
        if (ops_out) ops_out[i] = p->kernel_ops[i];
    }
    return SAETTA_OK;
}

int saetta_plan_build_where(saetta_plan *p, const char *const *keep, size_t n_keep, int barriers, saetta_built **out) {
    if (!p || !out || (n_keep && !keep)) return fail(SAETTA_ERR_BAD_ARG, "Plan::build_where: null pointer");
    if (!p->graph) return fail(SAETTA_ERR_BAD_ARG, "Plan::build_where: the plan has not been built");
    DeviceGuard guard(p->device);
    Recorded r;
    if (int rc = recorded_order(p->graph, r)) return rc;
    auto *b = new (std::nothrow) saetta_built();
    if (!b) return fail(SAETTA_ERR_NO_MEM, "Plan::build_where: host allocation");
    b->device = p->device, b->stream = p->stream;
    cudaError_t e = cudaGraphCreate(&b->graph, 0);
    if (e == cudaSuccess) e = cudaEventCreate(&b->t0);
    if (e == cudaSuccess) e = cudaEventCreate(&b->t1);
    if (e != cudaSuccess) {
        saetta_built_destroy(b);
        return cuda_fail(e, "Plan::build_where");
    }
    // For every recorded node, the nodes of the new graph that stand for "everything before it":
    // its own copy when it is kept, else what its own dependencies stand for.
    std::map<cudaGraphNode_t, std::vector<cudaGraphNode_t>> stands;
    int rc = SAETTA_OK;
    for (cudaGraphNode_t node : r.order) {
        std::vector<cudaGraphNode_t> before;
        for (cudaGraphNode_t d : r.deps[node])
            for (cudaGraphNode_t s : stands[d])
                if (std::find(before.begin(), before.end(), s) == before.end()) before.push_back(s);
        cudaGraphNodeType t;
        if ((e = cudaGraphNodeGetType(node, &t)) != cudaSuccess) break;
        cudaGraphNode_t copy = nullptr;
        if (t == cudaGraphNodeTypeKernel) {
            std::string name;
            cudaKernelNodeParams kp;
            if ((rc = kernel_name(node, name, kp))) break;
            bool kept = n_keep == 0;
            for (size_t i = 0; i < n_keep && !kept; i++) kept = keep[i] && name.find(keep[i]) != std::string::npos;
            if (kept) {
                // without the barriers a kernel waits for the copies before it, not for other kernels
                std::vector<cudaGraphNode_t> deps;
                for (cudaGraphNode_t s : before)
                    if (barriers || !b->is_kernel[s]) deps.push_back(s);
                if ((e = cudaGraphAddKernelNode(&copy, b->graph, deps.data(), deps.size(), &kp)) != cudaSuccess) break;
                b->is_kernel[copy] = true;
                b->kernels++;
            }
        } else if (t == cudaGraphNodeTypeMemcpy) {
            cudaMemcpy3DParms mp;
            if ((e = cudaGraphMemcpyNodeGetParams(node, &mp)) != cudaSuccess) break;
            if ((e = cudaGraphAddMemcpyNode(&copy, b->graph, before.data(), before.size(), &mp)) != cudaSuccess) break;
        } else if (t == cudaGraphNodeTypeMemset) {
            cudaMemsetParams mp;
            if ((e = cudaGraphMemsetNodeGetParams(node, &mp)) != cudaSuccess) break;
            if ((e = cudaGraphAddMemsetNode(&copy, b->graph, before.data(), before.size(), &mp)) != cudaSuccess) break;
        }
        if (copy) {
            b->is_kernel.emplace(copy, t == cudaGraphNodeTypeKernel);
            stands[node] = {copy};
        } else {
            stands[node] = before; // dropped (or an empty / event node): order passes through it
        }
    }
    if (e == cudaSuccess && !rc) e = cudaGraphInstantiate(&b->exec, b->graph, 0);
    if (e != cudaSuccess || rc) {
        saetta_built_destroy(b);
        return rc ? rc : cuda_fail(e, "Plan::build_where");
    }
    *out = b;
    return SAETTA_OK;
}

void saetta_built_destroy(saetta_built *b) {
    if (!b) return;
    DeviceGuard guard(b->device);
    if (b->exec) cudaGraphExecDestroy(b->exec);
    if (b->graph) cudaGraphDestroy(b->graph);
    if (b->t0) cudaEventDestroy(b->t0);
    if (b->t1) cudaEventDestroy(b->t1);
    delete b;
}

int saetta_built_len(const saetta_built *b, size_t *ops) {
    if (!b || !ops) return fail(SAETTA_ERR_BAD_ARG, "Built: null pointer");
    *ops = b->kernels;
    return SAETTA_OK;
}

// Built::run_timed: one replay on the plan's stream, waited for; the GPU's own time in milliseconds.
int saetta_built_run_timed(saetta_built *b, float *gpu_ms) {
    if (!b) return fail(SAETTA_ERR_BAD_ARG, "Built::run: null pointer");
    DeviceGuard guard(b->device);
    SAETTA_CUDA(cudaEventRecord(b->t0, b->stream));
    SAETTA_CUDA(cudaGraphLaunch(b->exec, b->stream));
    SAETTA_CUDA(cudaEventRecord(b->t1, b->stream));
    SAETTA_CUDA(cudaStreamSynchronize(b->stream));
    if (gpu_ms) SAETTA_CUDA(cudaEventElapsedTime(gpu_ms, b->t0, b->t1));
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
