// graph.cu: recording what is queued on a GPU's compute stream and replaying it as one submission - the CUDA-graph form
// of the reference's SYCL-graph hooks (kernels/llm/qwen35/q35.h:47-52, q35.cpp:508-551): begin starts recording (nothing
// runs), end finishes and instantiates, launch replays on the compute stream, free releases.
#include "ns_internal.cuh"

namespace {
struct NsGraph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};
}  // namespace

extern "C" {

int ns_q35_graph_begin(ns_gpu* g, void** out) {
    NS_TRY
    if (ns_enter(g, "ns_q35_graph_begin")) return -1;
    if (!out) return ns_fail("ns_q35_graph_begin: no out");
    NS_CUDA(cudaStreamBeginCapture(g->compute, cudaStreamCaptureModeThreadLocal), "ns_q35_graph_begin");
    *out = new NsGraph();
    return 0;
    NS_CATCH("ns_q35_graph_begin")
}

int ns_q35_graph_end(ns_gpu* g, void* h) {
    NS_TRY
    if (ns_enter(g, "ns_q35_graph_end")) return -1;
    NsGraph* gr = static_cast<NsGraph*>(h);
    if (!gr) return ns_fail("ns_q35_graph_end: no graph");
    NS_CUDA(cudaStreamEndCapture(g->compute, &gr->graph), "ns_q35_graph_end");
    NS_CUDA(cudaGraphInstantiate(&gr->exec, gr->graph, 0), "ns_q35_graph_end");
    return 0;
    NS_CATCH("ns_q35_graph_end")
}

int ns_q35_graph_launch(ns_gpu* g, void* h) {
    NS_TRY
    if (ns_enter(g, "ns_q35_graph_launch")) return -1;
    NsGraph* gr = static_cast<NsGraph*>(h);
    if (!gr || !gr->exec) return ns_fail("ns_q35_graph_launch: a graph not finished");
    NS_CUDA(cudaGraphLaunch(gr->exec, g->compute), "ns_q35_graph_launch");
    return 0;
    NS_CATCH("ns_q35_graph_launch")
}

void ns_q35_graph_free(void* h) {
    NsGraph* gr = static_cast<NsGraph*>(h);
    if (!gr) return;
    if (gr->exec) cudaGraphExecDestroy(gr->exec);
    if (gr->graph) cudaGraphDestroy(gr->graph);
    delete gr;
}

}  // extern "C"
