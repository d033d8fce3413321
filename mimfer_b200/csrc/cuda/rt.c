/*
 * Stand-alone CUDA runtime shim for the NVFP4 linear library.
 *
 * Plays the part of mimfer's src/cuda/cuda_rt.c for the few services the
 * launcher and the op-list engine use: two non-blocking streams (compute,
 * transfer), stream capture on the compute stream into an instantiated
 * graph, async copies, and the "capturing" flag the launchers consult so they
 * neither synchronise nor read back inside a capture
 * (include/mimfer/cuda_rt.h:86-94).  Process-global state for one device and
 * one host thread, as in the reference (src/cuda/cuda_rt.c:15-18).
 *
 * When the library is linked into a mimfer build, leave this file out: the
 * same symbols then come from mimfer's own runtime.
 */
#include "../core/core.h"
#include "../kernels/launch.h"
#include <cuda_runtime_api.h>
#include <stdlib.h>

static cudaStream_t g_stream[MM_ST_N];
static cudaEvent_t  g_t0, g_t1;
static cudaEvent_t *g_events;             /* ordering events, no timing: MM_N_EVENTS at init */
static int          g_n_events;
static int          g_ready, g_capturing, g_device = -1;

#define CK(call)                                                              \
    do {                                                                      \
        cudaError_t e_ = (call);                                              \
        if (e_ != cudaSuccess) {                                              \
            MM_LOGE("cuda: %s: %s", #call, cudaGetErrorString(e_));           \
            return MM_ERR_CUDA;                                               \
        }                                                                     \
    } while (0)

int mm_cuda_enabled(void) { return 1; }

mm_status mm_cuda_device_count(int *n_out)
{
    MM_REQUIRE(n_out, MM_ERR_STATE);
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    *n_out = n;
    return MM_OK;
}

mm_status mm_cuda_init(int device_ordinal)
{
    int dev = device_ordinal < 0 ? 0 : device_ordinal;
    if (g_ready)
        return dev == g_device ? MM_OK : MM_ERR_BUSY;
    struct cudaDeviceProp prop;
    CK(cudaSetDevice(dev));
    CK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) {
        MM_LOGE("device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major,
                prop.minor);
        return MM_ERR_DEVICE;
    }
    CK(cudaStreamCreateWithFlags(&g_stream[MM_ST_COMPUTE], cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&g_stream[MM_ST_XFER], cudaStreamNonBlocking));
    CK(cudaEventCreate(&g_t0));
    CK(cudaEventCreate(&g_t1));
    g_device = dev;
    g_ready = 1;
    return mmb_event_pool_reserve(MM_N_EVENTS);
}

/* Grow the event pool to at least n events (set-up time only). */
mm_status mmb_event_pool_reserve(int n)
{
    MM_REQUIRE(g_ready && n > 0, MM_ERR_STATE);
    if (n <= g_n_events)
        return MM_OK;
    cudaEvent_t *ev = (cudaEvent_t *)realloc(g_events, (size_t)n * sizeof *ev);
    if (!ev)
        return MM_ERR_NOMEM;
    g_events = ev;
    while (g_n_events < n) {
        CK(cudaEventCreateWithFlags(&g_events[g_n_events], cudaEventDisableTiming));
        g_n_events++;
    }
    return MM_OK;
}

mm_status mm_event_record(int ev, mm_stream_id st)
{
    MM_REQUIRE(g_ready && ev >= 0 && ev < g_n_events && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaEventRecord(g_events[ev], g_stream[st]));
    return MM_OK;
}

mm_status mm_event_wait(int ev, mm_stream_id st)
{
    MM_REQUIRE(g_ready && ev >= 0 && ev < g_n_events && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaStreamWaitEvent(g_stream[st], g_events[ev], 0));
    return MM_OK;
}

mm_status mm_cuda_shutdown(void)
{
    if (!g_ready)
        return MM_OK;
    cudaEventDestroy(g_t0);
    cudaEventDestroy(g_t1);
    for (int i = 0; i < g_n_events; i++)
        cudaEventDestroy(g_events[i]);
    free(g_events);
    g_events = NULL;
    g_n_events = 0;
    cudaStreamDestroy(g_stream[MM_ST_COMPUTE]);
    cudaStreamDestroy(g_stream[MM_ST_XFER]);
    mmb_launcher_reset();       /* status word, workspace and kernel attributes belong to this device */
    g_ready = 0;
    g_device = -1;
    return MM_OK;
}

void *mm_cuda_stream_raw(mm_stream_id id)
{
    return (g_ready && (int)id >= 0 && id < MM_ST_N) ? (void *)g_stream[id] : NULL;
}

int mm_cuda_capturing(void) { return g_capturing; }

mm_status mm_stream_sync(mm_stream_id st)
{
    MM_REQUIRE(g_ready && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaStreamSynchronize(g_stream[st]));
    return MM_OK;
}

mm_status mm_h2d_async(void *dst, const void *src, size_t n, mm_stream_id st)
{
    MM_REQUIRE(g_ready && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, g_stream[st]));
    return MM_OK;
}

mm_status mm_d2h_async(void *dst, const void *src, size_t n, mm_stream_id st)
{
    MM_REQUIRE(g_ready && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, g_stream[st]));
    return MM_OK;
}

mm_status mm_mset_async(void *dst, int value, size_t n, mm_stream_id st)
{
    MM_REQUIRE(g_ready && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaMemsetAsync(dst, value, n, g_stream[st]));
    return MM_OK;
}

/* ---- graphs --------------------------------------------------------------- */
struct mm_graph {
    cudaGraphExec_t exec;
    int             have_exec;
};

mm_status mm_graph_create(mm_graph **out)
{
    MM_REQUIRE(out, MM_ERR_STATE);
    *out = (mm_graph *)calloc(1, sizeof(mm_graph));
    return *out ? MM_OK : MM_ERR_NOMEM;
}

mm_status mm_graph_capture_begin(mm_graph *g)
{
    MM_REQUIRE(g && g_ready, MM_ERR_STATE);
    MM_REQUIRE(!g_capturing, MM_ERR_BUSY);            /* one capture at a time */
    CK(cudaStreamBeginCapture(g_stream[MM_ST_COMPUTE], cudaStreamCaptureModeThreadLocal));
    g_capturing = 1;
    return MM_OK;
}

mm_status mm_graph_commit(mm_graph *g, const void *window_base, size_t window_bytes,
                          int hit_ratio_pct)
{
    /* The L2 access-policy window of the reference (src/cuda/cuda_rt.c:163-251)
     * is accepted and ignored: on B200 the decode weights stream once per step
     * and do not fit L2. */
    (void)window_base; (void)window_bytes; (void)hit_ratio_pct;
    MM_REQUIRE(g && g_capturing, MM_ERR_STATE);
    cudaGraph_t graph = NULL;
    cudaError_t e = cudaStreamEndCapture(g_stream[MM_ST_COMPUTE], &graph);
    g_capturing = 0;
    if (e != cudaSuccess || !graph) {
        MM_LOGE("cuda: end capture: %s", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return MM_ERR_CUDA;
    }
    if (g->have_exec) {
        cudaGraphExecDestroy(g->exec);
        g->have_exec = 0;
    }
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        MM_LOGE("cuda: graph instantiate: %s", cudaGetErrorString(e));
        return MM_ERR_CUDA;
    }
    g->have_exec = 1;
    return MM_OK;
}

mm_status mm_graph_launch(mm_graph *g, mm_stream_id st)
{
    MM_REQUIRE(g && g->have_exec && g_ready && (int)st >= 0 && st < MM_ST_N, MM_ERR_STATE);
    CK(cudaGraphLaunch(g->exec, g_stream[st]));
    return MM_OK;
}

void mm_graph_destroy(mm_graph *g)
{
    if (!g)
        return;
    if (g->have_exec)
        cudaGraphExecDestroy(g->exec);
    free(g);
}

/* ---- timing on the compute stream ------------------------------------------ */
mm_status mm_time_begin(void)
{
    MM_REQUIRE(g_ready, MM_ERR_STATE);
    CK(cudaEventRecord(g_t0, g_stream[MM_ST_COMPUTE]));
    return MM_OK;
}

mm_status mm_time_end(float *ms_out)
{
    MM_REQUIRE(g_ready && ms_out, MM_ERR_STATE);
    CK(cudaEventRecord(g_t1, g_stream[MM_ST_COMPUTE]));
    CK(cudaEventSynchronize(g_t1));
    CK(cudaEventElapsedTime(ms_out, g_t0, g_t1));
    return MM_OK;
}
