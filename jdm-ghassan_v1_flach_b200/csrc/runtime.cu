// Process-wide state of the library: last error, current stream, cached
// workspaces, device utilities (the gai::cuda::* functions of the reference,
// cuda/cuda_utils.cu) and the recorded-only toggles.
#include <cstring>
#include <mutex>
#include <string>

#include <nvtx3/nvToolsExt.h>

#include <vector>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[512] = "";
static cudaStream_t g_stream = nullptr;   // legacy default stream, as in the reference
static Workspace g_ws[WS_COUNT];
static int g_sms = 0;
unsigned long long g_kernel_launches = 0;
static bool g_fp16_gemm = false, g_bf16_gemm = false;

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_status(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? B200_ENOMEM : B200_ECUDA;
}

cudaStream_t stream() { return g_stream; }

int num_sms() {
    if (g_sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            g_sms = n;
        else
            g_sms = 148;
    }
    return g_sms;
}

// Bumped whenever a workspace's device address stops being valid (reallocation or
// release): what a captured CUDA graph compares against before it is replayed.
static unsigned long long g_ws_generation = 0;
unsigned long long workspace_generation() { return g_ws_generation; }

int Workspace::ensure(size_t need, void** out) {
    if (need > bytes) {
        ++g_ws_generation;
        if (ptr) {
            B200_CUDA(cudaFree(ptr));
            ptr = nullptr;
            bytes = 0;
        }
        const size_t mb = (size_t)1 << 20;
        const size_t rounded = (need + mb - 1) / mb * mb;
        B200_CUDA(cudaMalloc(&ptr, rounded));
        bytes = rounded;
    }
    *out = ptr;
    return B200_OK;
}

void Workspace::release() {
    if (ptr) ++g_ws_generation;
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
}

Workspace& workspace(int which) { return g_ws[which]; }

// ---- side stream ----------------------------------------------------------
// Work that does not depend on what the current stream is doing (the shared expert of an
// MoE layer next to the routing of the same tokens) is enqueued on a second stream between
// side_begin() and side_end(); side_wait() makes the current stream wait for it.  Events
// only: legal inside a stream capture (the side stream joins the capture and rejoins).
static cudaStream_t g_side = nullptr, g_side_prev = nullptr;
static cudaEvent_t g_side_fork = nullptr, g_side_join = nullptr;
int side_begin() {
    if (!g_side) {
        B200_CUDA(cudaStreamCreateWithFlags(&g_side, cudaStreamNonBlocking));
        B200_CUDA(cudaEventCreateWithFlags(&g_side_fork, cudaEventDisableTiming));
        B200_CUDA(cudaEventCreateWithFlags(&g_side_join, cudaEventDisableTiming));
    }
    B200_CUDA(cudaEventRecord(g_side_fork, g_stream));
    B200_CUDA(cudaStreamWaitEvent(g_side, g_side_fork, 0));
    g_side_prev = g_stream;
    g_stream = g_side;
    return B200_OK;
}
int side_end() {
    g_stream = g_side_prev;
    B200_CUDA(cudaEventRecord(g_side_join, g_side));
    return B200_OK;
}
int side_wait() {
    B200_CUDA(cudaStreamWaitEvent(g_stream, g_side_join, 0));
    return B200_OK;
}

// ---- phase timers ------------------------------------------------------------------
// Intervals are (start event, stop event, phase id); events come from a free list and go
// back to it when a report has read them.
struct PhaseInterval { cudaEvent_t s, e; int ph; bool open; };
static std::vector<PhaseInterval> g_intervals;
static std::vector<cudaEvent_t> g_free_events;
static int phase_event(cudaEvent_t* ev) {
    if (!g_free_events.empty()) {
        *ev = g_free_events.back();
        g_free_events.pop_back();
        return B200_OK;
    }
    B200_CUDA(cudaEventCreate(ev));
    return B200_OK;
}
static int phase_close_open() {
    if (!g_intervals.empty() && g_intervals.back().open) {
        B200_CUDA(cudaEventRecord(g_intervals.back().e, g_stream));
        g_intervals.back().open = false;
        nvtxRangePop();
    }
    return B200_OK;
}

void nvtx_push(const char* name) { nvtxRangePushA(name); }
void nvtx_pop() { nvtxRangePop(); }

}  // namespace b200

using namespace b200;

extern "C" {

int b200_phase_start(int phase) {
    B200_REQUIRE(phase >= 0 && phase < 8, "phase_start: phase id %d outside 0 .. 7", phase);
    int rc = phase_close_open();
    if (rc) return rc;
    PhaseInterval it{nullptr, nullptr, phase, true};
    if ((rc = phase_event(&it.s)) || (rc = phase_event(&it.e))) return rc;
    B200_CUDA(cudaEventRecord(it.s, g_stream));
    g_intervals.push_back(it);
    char name[32];
    snprintf(name, sizeof(name), "b200.phase%d", phase);
    nvtxRangePushA(name);
    return B200_OK;
}
int b200_phase_stop(int) { return phase_close_open(); }
int b200_phase_reset(void) {
    if (!g_intervals.empty() && g_intervals.back().open) nvtxRangePop();
    for (PhaseInterval& it : g_intervals) {
        g_free_events.push_back(it.s);
        g_free_events.push_back(it.e);
    }
    g_intervals.clear();
    return B200_OK;
}
int b200_phase_shutdown(void) {
    b200_phase_reset();
    for (cudaEvent_t ev : g_free_events) cudaEventDestroy(ev);
    g_free_events.clear();
    return B200_OK;
}
int b200_phase_report(double* ms, int n_phases) {
    B200_REQUIRE(ms && n_phases >= 1 && n_phases <= 8, "phase_report: bad arguments");
    std::vector<PhaseInterval> keep;
    for (PhaseInterval& it : g_intervals) {
        bool done = false;
        if (!it.open && cudaEventQuery(it.e) == cudaSuccess) {
            float d = 0.0f;
            if (cudaEventElapsedTime(&d, it.s, it.e) == cudaSuccess) {
                if (it.ph < n_phases) ms[it.ph] += (double)d;
                done = true;
            }
        }
        cudaGetLastError();      // a query of a running event is not an error of ours
        if (done) {
            g_free_events.push_back(it.s);
            g_free_events.push_back(it.e);
        } else {
            keep.push_back(it);
        }
    }
    g_intervals.swap(keep);
    return B200_OK;
}

const char* b200_last_error(void) { return g_err; }
int b200_version(void) { return 100; }
uint64_t b200_kernel_launches(void) { return g_kernel_launches; }

int b200_device_count(int* count) {
    B200_REQUIRE(count, "device_count: null pointer");
    B200_CUDA(cudaGetDeviceCount(count));
    return B200_OK;
}
int b200_device_info(int* index, char* name, int name_cap, int* cc_major, int* cc_minor,
                     size_t* total_mem, size_t* free_mem) {
    static bool selected = false;
    if (!selected) {
        // one process per GPU: LOCAL_RANK picks the device, like the reference's probe
        const char* lr = getenv("LOCAL_RANK");
        int count = 0;
        B200_CUDA(cudaGetDeviceCount(&count));
        if (lr && count > 0) B200_CUDA(cudaSetDevice(atoi(lr) % count));
        selected = true;
    }
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    B200_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (index) *index = dev;
    if (name && name_cap > 0) snprintf(name, (size_t)name_cap, "%s", prop.name);
    if (cc_major) *cc_major = prop.major;
    if (cc_minor) *cc_minor = prop.minor;
    size_t fr = 0, tot = 0;
    B200_CUDA(cudaMemGetInfo(&fr, &tot));
    if (total_mem) *total_mem = tot;
    if (free_mem) *free_mem = fr;
    return B200_OK;
}
int b200_shutdown(void) { return b200_free_workspaces(); }
int b200_malloc_device(void** ptr, size_t nbytes) {
    B200_REQUIRE(ptr, "malloc_device: null pointer");
    *ptr = nullptr;
    if (nbytes == 0) return B200_OK;
    B200_CUDA(cudaMalloc(ptr, nbytes));
    return B200_OK;
}
int b200_free_device(void* ptr) {
    if (ptr) B200_CUDA(cudaFree(ptr));
    return B200_OK;
}
int b200_memset_zero(void* ptr, size_t nbytes) {
    if (!ptr || nbytes == 0) return B200_OK;
    B200_CUDA(cudaMemsetAsync(ptr, 0, nbytes, stream()));
    return B200_OK;
}
int b200_is_device_memory(const void* ptr, int* yes) {
    B200_REQUIRE(yes, "is_device_memory: null pointer");
    cudaPointerAttributes at;
    const cudaError_t e = cudaPointerGetAttributes(&at, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *yes = 0;
        return B200_OK;
    }
    *yes = (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) ? 1 : 0;
    return B200_OK;
}
int b200_copy(void* dst, int dst_is_device, const void* src, int src_is_device, size_t nbytes) {
    if (nbytes == 0) return B200_OK;
    B200_REQUIRE(dst && src, "copy: null pointer");
    const cudaMemcpyKind kind = dst_is_device ? (src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice)
                                              : (src_is_device ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost);
    // Ordered on the library's stream, then completed before returning, like the
    // reference's blocking cudaMemcpy on stream 0.
    B200_CUDA(cudaMemcpyAsync(dst, src, nbytes, kind, stream()));
    if (kind != cudaMemcpyDeviceToDevice) B200_CUDA(cudaStreamSynchronize(stream()));
    return B200_OK;
}
int b200_synchronize(void) {
    B200_CUDA(cudaDeviceSynchronize());
    return b200::stream_status_check("synchronize");    // surfaces a bounded wait that ran out
}
int b200_free_bytes_live(size_t* bytes) {
    B200_REQUIRE(bytes, "free_bytes_live: null pointer");
    size_t total = 0;
    B200_CUDA(cudaMemGetInfo(bytes, &total));
    return B200_OK;
}
int b200_set_stream(void* s) {
    g_stream = static_cast<cudaStream_t>(s);
    return B200_OK;
}

int b200_set_fp16_gemm(int on) { g_fp16_gemm = on != 0; return B200_OK; }
int b200_fp16_gemm_enabled(void) { return g_fp16_gemm ? 1 : 0; }
int b200_set_bf16_gemm(int on) { g_bf16_gemm = on != 0; return B200_OK; }
int b200_bf16_gemm_enabled(void) { return g_bf16_gemm ? 1 : 0; }
int b200_set_moe_jitter(float j) {
    if (j != 0.0f)
        return fail(B200_EUNSUPPORTED, "set_moe_jitter: router noise is a training feature; the "
                                       "inference backend only accepts 0");
    return B200_OK;
}
int b200_set_moe_jitter_seed(uint64_t) { return B200_OK; }

int b200_free_workspace(void) { workspace(WS_LINEAR).release(); workspace(WS_ATTN).release(); return B200_OK; }
int b200_moe_free_workspace(void) { workspace(WS_MOE).release(); return B200_OK; }
int b200_mamba_free_workspace(void) { workspace(WS_MAMBA).release(); return B200_OK; }
int b200_free_sampling_workspace(void) { workspace(WS_SAMPLE).release(); return B200_OK; }
int b200_free_workspaces(void) {
    for (int i = 0; i < WS_COUNT; ++i) workspace(i).release();
    return b200_free_quant_scratch();
}
int b200_reserve_workspaces(size_t gemm_bytes, size_t moe_bytes) {
    void* p;
    if (gemm_bytes) { int rc = workspace(WS_LINEAR).ensure(gemm_bytes, &p); if (rc) return rc; }
    if (moe_bytes) { int rc = workspace(WS_MOE).ensure(moe_bytes, &p); if (rc) return rc; }
    return B200_OK;
}
int b200_moe_reserve_workspace(size_t bytes) {
    void* p;
    return bytes ? workspace(WS_MOE).ensure(bytes, &p) : B200_OK;
}
size_t b200_pool_bytes(void) { return workspace(WS_LINEAR).bytes + workspace(WS_ATTN).bytes + workspace(WS_MAMBA).bytes; }
size_t b200_moe_pool_bytes(void) { return workspace(WS_MOE).bytes; }

int b200_training_op_unsupported(const char* name) {
    return fail(B200_EUNSUPPORTED, "%s: training op not provided by the B200 inference backend",
                name ? name : "?");
}

}  // extern "C"
