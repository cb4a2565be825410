// Side streams and captured step graphs for compiled segments.
//
// A segment's Execute is the same launches every time for a given row count: kernels, copies of the outputs to
// page-locked staging. Issued from the host one by one, a decode step of a few dozen launches is bound by the host's
// launch rate; captured once into a CUDA graph and replayed, it is one call. Inside the capture a second stream carries
// the device-to-host copies, forked after the kernel that produces each output and joined at the end, so the copy
// engine works while the later kernels run. The reference's Vulkan provider records a segment's command buffer once and
// re-submits it (ICompiledSegment: "Implementations may run asynchronously until an output is read",
// src/Sharplight.Core/Runtime/ICompiledSegment.cs:11-12); this is the CUDA form of that.
#include "../../include/sharplight_cuda.h"

#include "handles.cuh"

#include <new>
#include <string>

struct slc_graph
{
    slc_device *dev = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

namespace {

thread_local std::string t_graph_error;

slc_result g_fail(slc_result code, const std::string &msg)
{
    t_graph_error = msg;
    return code;
}

slc_result g_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return SLC_OK;
    return g_fail(SLC_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

extern "C" {

const char *slc_graph_last_error(void) { return t_graph_error.c_str(); }

slc_result slc_stream_create(slc_device *d, void **out_stream)
{
    if (!d || !out_stream) return g_fail(SLC_ERR_INVALID_ARGUMENT, "device or out_stream is null");
    *out_stream = nullptr;
    slc_result r = g_cuda(cudaSetDevice(d->index), "cudaSetDevice");
    if (r != SLC_OK) return r;
    cudaStream_t s = nullptr;
    r = g_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    if (r != SLC_OK) return r;
    *out_stream = s;
    return SLC_OK;
}

void slc_stream_destroy(slc_device *d, void *stream)
{
    if (!d || !stream) return;
    cudaSetDevice(d->index);
    cudaStreamDestroy((cudaStream_t)stream);
}

slc_result slc_stream_wait(slc_device *d, void *waiter, void *signal)
{
    if (!d) return g_fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    cudaStream_t w = waiter ? (cudaStream_t)waiter : d->stream, s = signal ? (cudaStream_t)signal : d->stream;
    if (w == s) return SLC_OK;
    slc_result r = g_cuda(cudaSetDevice(d->index), "cudaSetDevice");
    if (r != SLC_OK) return r;
    cudaEvent_t ev = nullptr;
    r = g_cuda(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreateWithFlags");
    if (r != SLC_OK) return r;
    // Inside a capture the event becomes part of the graph being built: it is kept until the device closes. Outside,
    // it has done its work once the wait is enqueued (destroying an event that streams still wait on is safe: the
    // resources go when the work completes), so a long-running host does not accumulate events.
    cudaStreamCaptureStatus cap_w = cudaStreamCaptureStatusNone, cap_s = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(w, &cap_w);
    cudaStreamIsCapturing(s, &cap_s);
    const bool capturing = cap_w != cudaStreamCaptureStatusNone || cap_s != cudaStreamCaptureStatusNone;
    cudaError_t e = cudaEventRecord(ev, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(w, ev, 0);
    if (capturing) d->events.push_back(ev);
    else cudaEventDestroy(ev);
    return g_cuda(e, "cudaEventRecord / cudaStreamWaitEvent");
}

slc_result slc_graph_begin(slc_device *d, void *stream)
{
    if (!d) return g_fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    slc_result r = g_cuda(cudaSetDevice(d->index), "cudaSetDevice");
    if (r != SLC_OK) return r;
    return g_cuda(cudaStreamBeginCapture(stream ? (cudaStream_t)stream : d->stream, cudaStreamCaptureModeThreadLocal),
                  "cudaStreamBeginCapture");
}

slc_result slc_graph_end(slc_device *d, void *stream, slc_graph **out)
{
    if (!d || !out) return g_fail(SLC_ERR_INVALID_ARGUMENT, "device or out is null");
    *out = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream ? (cudaStream_t)stream : d->stream, &graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return g_fail(SLC_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
    }
    slc_graph *g = new (std::nothrow) slc_graph();
    if (!g) {
        cudaGraphDestroy(graph);
        return g_fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    }
    g->dev = d;
    g->graph = graph;
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete g;
        return g_fail(SLC_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    }
    *out = g;
    return SLC_OK;
}

slc_result slc_graph_launch(slc_graph *g, void *stream)
{
    if (!g) return g_fail(SLC_ERR_INVALID_ARGUMENT, "graph is null");
    slc_result r = g_cuda(cudaSetDevice(g->dev->index), "cudaSetDevice");
    if (r != SLC_OK) return r;
    return g_cuda(cudaGraphLaunch(g->exec, stream ? (cudaStream_t)stream : g->dev->stream), "cudaGraphLaunch");
}

void slc_graph_destroy(slc_graph *g)
{
    if (!g) return;
    cudaSetDevice(g->dev->index);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
}

}  // extern "C"
