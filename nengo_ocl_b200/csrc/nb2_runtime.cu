// Device runtime behind the C ABI: memory, streams, events, CUDA-graph
// capture/replay and error reporting.  Replaces what the reference obtains
// from PyOpenCL (context/queue creation nengo_ocl/simulator.py:209-219,
// to_device / Array.get / enqueue_copy in nengo_ocl/clraggedarray.py:36-62,
// 128-196, and the per-plan enqueue loop nengo_ocl/plan.py:85-149).
#include <stdarg.h>
#include <string.h>

#include <stdlib.h>
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

static thread_local char g_err[1024] = "";

void nb2_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" {

const char* nb2_last_error(void) { return g_err; }

int nb2_abi_version(void) { return NB2_ABI_VERSION; }

// -1: not decided yet (first use reads the environment)
static int g_programmatic_launch = -1;

int nb2_programmatic_launch_enabled() {
  if (g_programmatic_launch < 0) {
    const char* env = getenv("NENGO_B200_PDL");
    g_programmatic_launch = (env != NULL && env[0] == '0') ? 0 : 1;
  }
  return g_programmatic_launch;
}

int nb2_set_programmatic_launch(int enabled) {
  g_programmatic_launch = enabled ? 1 : 0;
  return NB2_OK;
}

int nb2_device_count(int* count) {
  NB2_REQUIRE(count != NULL, "count");
  NB2_CUDA(cudaGetDeviceCount(count));
  return NB2_OK;
}

int nb2_set_device(int ordinal) {
  NB2_CUDA(cudaSetDevice(ordinal));
  return NB2_OK;
}

int nb2_device_info(int ordinal, int* sm_count, int* max_threads_per_block,
                    size_t* global_mem, size_t* shared_mem_per_block_optin,
                    int* cc_major, int* cc_minor) {
  cudaDeviceProp p;
  NB2_CUDA(cudaGetDeviceProperties(&p, ordinal));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (max_threads_per_block) *max_threads_per_block = p.maxThreadsPerBlock;
  if (global_mem) *global_mem = p.totalGlobalMem;
  if (shared_mem_per_block_optin) *shared_mem_per_block_optin = p.sharedMemPerBlockOptin;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return NB2_OK;
}

int nb2_malloc(void** dptr, size_t bytes) {
  NB2_REQUIRE(dptr != NULL, "dptr");
  *dptr = NULL;
  // whole 256-byte granules: a valid, distinct pointer for empty arrays, and kernels that
  // stage 16-byte-aligned windows may read up to the next 16-byte boundary past the end
  bytes = bytes ? (bytes + 255) & ~(size_t)255 : 256;
  NB2_CUDA(cudaMalloc(dptr, bytes));
  return NB2_OK;
}

int nb2_free(void* dptr) {
  if (dptr) NB2_CUDA(cudaFree(dptr));
  return NB2_OK;
}

int nb2_host_alloc(void** hptr, size_t bytes) {
  NB2_REQUIRE(hptr != NULL, "hptr");
  NB2_CUDA(cudaMallocHost(hptr, bytes ? bytes : 16));
  return NB2_OK;
}

int nb2_host_free(void* hptr) {
  if (hptr) NB2_CUDA(cudaFreeHost(hptr));
  return NB2_OK;
}

int nb2_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream, int sync) {
  if (bytes == 0) return NB2_OK;
  NB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, nb2_stream(stream)));
  if (sync) NB2_CUDA(cudaStreamSynchronize(nb2_stream(stream)));
  return NB2_OK;
}

int nb2_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream, int sync) {
  if (bytes == 0) return NB2_OK;
  NB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, nb2_stream(stream)));
  if (sync) NB2_CUDA(cudaStreamSynchronize(nb2_stream(stream)));
  return NB2_OK;
}

int nb2_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return NB2_OK;
  NB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, nb2_stream(stream)));
  return NB2_OK;
}

int nb2_memset(void* dst, int byte_value, size_t bytes, void* stream) {
  if (bytes == 0) return NB2_OK;
  NB2_CUDA(cudaMemsetAsync(dst, byte_value, bytes, nb2_stream(stream)));
  return NB2_OK;
}

int nb2_stream_create(void** stream) {
  NB2_REQUIRE(stream != NULL, "stream");
  cudaStream_t s;
  NB2_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = (void*)s;
  return NB2_OK;
}

int nb2_stream_destroy(void* stream) {
  if (stream) NB2_CUDA(cudaStreamDestroy(nb2_stream(stream)));
  return NB2_OK;
}

int nb2_stream_sync(void* stream) {
  NB2_CUDA(cudaStreamSynchronize(nb2_stream(stream)));
  return NB2_OK;
}

int nb2_device_sync(void) {
  NB2_CUDA(cudaDeviceSynchronize());
  return NB2_OK;
}

int nb2_event_create(void** event) {
  NB2_REQUIRE(event != NULL, "event");
  cudaEvent_t e;
  NB2_CUDA(cudaEventCreate(&e));
  *event = (void*)e;
  return NB2_OK;
}

int nb2_event_destroy(void* event) {
  if (event) NB2_CUDA(cudaEventDestroy((cudaEvent_t)event));
  return NB2_OK;
}

int nb2_event_record(void* event, void* stream) {
  NB2_CUDA(cudaEventRecord((cudaEvent_t)event, nb2_stream(stream)));
  return NB2_OK;
}

int nb2_stream_wait_event(void* stream, void* event) {
  NB2_CUDA(cudaStreamWaitEvent(nb2_stream(stream), (cudaEvent_t)event, 0));
  return NB2_OK;
}

int nb2_event_sync(void* event) {
  NB2_CUDA(cudaEventSynchronize((cudaEvent_t)event));
  return NB2_OK;
}

int nb2_event_elapsed_ms(void* start, void* stop, float* ms) {
  NB2_REQUIRE(ms != NULL, "ms");
  NB2_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return NB2_OK;
}

// ---- CUDA graph capture / replay ------------------------------------------
int nb2_graph_begin(void* stream) {
  // relaxed: an allocation or a free made by the host while the stream captures (e.g. by a
  // garbage collector) does not invalidate the capture
  NB2_CUDA(cudaStreamBeginCapture(nb2_stream(stream), cudaStreamCaptureModeRelaxed));
  return NB2_OK;
}

int nb2_graph_end(void* stream, void** graph_exec) {
  NB2_REQUIRE(graph_exec != NULL, "graph_exec");
  cudaGraph_t graph = NULL;
  NB2_CUDA(cudaStreamEndCapture(nb2_stream(stream), &graph));
  cudaGraphExec_t exec = NULL;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    nb2_set_error("cudaGraphInstantiate -> %s", cudaGetErrorString(e));
    return NB2_ERR_CUDA;
  }
  *graph_exec = (void*)exec;
  return NB2_OK;
}

int nb2_graph_abort(void* stream) {
  cudaGraph_t graph = NULL;
  cudaStreamEndCapture(nb2_stream(stream), &graph);
  if (graph) cudaGraphDestroy(graph);
  cudaGetLastError();
  return NB2_OK;
}

int nb2_graph_launch(void* graph_exec, void* stream, int n_times) {
  NB2_REQUIRE(graph_exec != NULL, "graph_exec");
  for (int i = 0; i < n_times; ++i)
    NB2_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, nb2_stream(stream)));
  return NB2_OK;
}

int nb2_graph_destroy(void* graph_exec) {
  if (graph_exec) NB2_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  return NB2_OK;
}

// ---- peer access for the multi-GPU exchange -------------------------------
int nb2_ipc_get_handle(void* dptr, void* handle64) {
  NB2_REQUIRE(handle64 != NULL, "handle64");
  cudaIpcMemHandle_t h;
  NB2_CUDA(cudaIpcGetMemHandle(&h, dptr));
  memcpy(handle64, &h, sizeof(h));
  return NB2_OK;
}

int nb2_ipc_open_handle(const void* handle64, void** dptr) {
  NB2_REQUIRE(handle64 != NULL && dptr != NULL, "handle64/dptr");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  NB2_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
  return NB2_OK;
}

int nb2_ipc_close_handle(void* dptr) {
  if (dptr) NB2_CUDA(cudaIpcCloseMemHandle(dptr));
  return NB2_OK;
}

}  // extern "C"
