// Expert-parallel MoE layer over peer memory: the host logic and the exchange kernels
// behind include/b200ep.h.  The compute steps are the single-GPU layer's building blocks
// (moe.cu, moe_grouped.cu, gemm_umma.cu); what is new here is how rows travel: every rank
// stores straight into its peers' blocks over NVLink (plain 16-byte stores), publishes an
// epoch number in a flag word behind a system-scope fence, and the consumer polls that word
// with a bounded wait.  No collective library, no host synchronisation, no TMA.
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/b200ep.h"
#include "gemm.cuh"
#include "linear.cuh"

namespace b200 {

constexpr int EP_MAXW = B200_EP_MAX_WORLD;
constexpr uint32_t EP_SPIN_DEFAULT = 1u << 24;      // polls of ~100 ns each: a couple of seconds

// Control words at the start of every rank's block.  flag_*[s] is written by rank s only.
struct EpCtrl {
    uint32_t flag_dispatch[EP_MAXW];   // rows + header of this pass have arrived from rank s
    uint32_t flag_return[EP_MAXW];     // rank s has returned the results of my rows
    uint32_t flag_gather[EP_MAXW];     // rank s has stored its output slice
    uint32_t done[4];                  // local: CTAs finished, per exchange kernel
    uint32_t pad[12];
};
static_assert(sizeof(EpCtrl) == 256, "control block layout");

// What the kernels need to know; passed by value.
struct EpDev {
    int rank, world, nl, cap, d;
    char* const* peers;                // device array [world] of block base addresses (peers[rank] = own)
    size_t off_hdr, off_rows, off_y, off_out;
    int* status;
    uint32_t spin_limit;
    // number of the pass in flight, in device memory so that a captured pass can be replayed:
    // every kernel reads it, the pass's last wait advances it
    uint32_t* epoch;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// After a CTA's peer stores: true in thread 0 of the grid's last CTA to get here (which then
// publishes the flags).  Every thread fences its own stores first.
__device__ __forceinline__ bool grid_last_cta(uint32_t* counter) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x != 0) return false;
    const uint32_t total = gridDim.x * gridDim.y;
    const uint32_t prev = atomicAdd(counter, 1u);
    if (prev + 1 != total) return false;
    *counter = 0;
    __threadfence_system();
    return true;
}
__device__ __forceinline__ EpCtrl* ctrl_of(const EpDev& e, int r) { return reinterpret_cast<EpCtrl*>(e.peers[r]); }
__device__ __forceinline__ int32_t* hdr_of(const EpDev& e, int r, int src) {
    return reinterpret_cast<int32_t*>(e.peers[r] + e.off_hdr) + (size_t)src * (e.nl + 2);
}

// x [n, d] fp32 (my token slice), grouped [NK] (slot numbers sorted by expert; slot / K is the
// token), offsets [ne + 1]: row i of that order is rounded to fp16 (clamped, as the packing of
// the single-GPU layer does) and stored into region `rank` of the receive buffer of the rank
// that owns its expert; header = rows per local expert, first row in my order, rows sent.
// One warp per row.
__global__ void __launch_bounds__(256) ep_pack_dispatch_kernel(EpDev e, const float* __restrict__ x,
                                                               const int32_t* __restrict__ grouped, int K,
                                                               const int32_t* __restrict__ offsets, int64_t NK) {
    const uint32_t epoch = *e.epoch;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < NK; i += nwarps) {
        int r = 0;
        while (r + 1 < e.world && i >= offsets[(r + 1) * e.nl]) ++r;
        const int64_t j = i - offsets[r * e.nl];
        if (j >= e.cap) continue;
        __half* dst = reinterpret_cast<__half*>(e.peers[r] + e.off_rows) + ((int64_t)e.rank * e.cap + j) * e.d;
        const float* src = x + (int64_t)(grouped[i] / K) * e.d;
        for (int k = lane * 8; k < e.d; k += 256) {
            const float4 a = *reinterpret_cast<const float4*>(src + k);
            const float4 b = *reinterpret_cast<const float4*>(src + k + 4);
            auto cl = [](float v) { return fminf(fmaxf(v, -65504.0f), 65504.0f); };
            __half2 h[4] = {__floats2half2_rn(cl(a.x), cl(a.y)), __floats2half2_rn(cl(a.z), cl(a.w)),
                            __floats2half2_rn(cl(b.x), cl(b.y)), __floats2half2_rn(cl(b.z), cl(b.w))};
            *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<uint4*>(h);
        }
    }
    if (blockIdx.x == 0) {
        const int per = e.nl + 2;
        for (int t = threadIdx.x; t < e.world * per; t += blockDim.x) {
            const int r = t / per, f = t - r * per;
            const int lo = offsets[r * e.nl], hi = offsets[(r + 1) * e.nl];
            int val;
            if (f < e.nl) {
                const int a = min(offsets[r * e.nl + f] - lo, e.cap), b = min(offsets[r * e.nl + f + 1] - lo, e.cap);
                val = b - a;
            } else if (f == e.nl) {
                val = lo;
            } else {
                val = min(hi - lo, e.cap);
                if (hi - lo > e.cap) atomicExch(e.status, 1);
            }
            hdr_of(e, r, e.rank)[f] = val;
        }
    }
    if (grid_last_cta(&ctrl_of(e, e.rank)->done[0]))
        for (int r = 0; r < e.world; ++r) st_release_sys(&ctrl_of(e, r)->flag_dispatch[e.rank], epoch);
}

// Bounded wait until every rank's flag has reached `epoch`.  which: 0 dispatch, 1 return,
// 2 gather.  With goff / gmap (dispatch only) the headers become the group list of the
// expert GEMMs: per sender nl groups (its rows per local expert, in arrival order) and one
// gap group (mapped to -1) up to the end of the sender's region.
// gc[g]: where group g's result rows go - the sender's y buffer at the position its header
// named - as a base to which the GEMM adds (row of the receive buffer) * d.
__global__ void ep_wait_kernel(EpDev e, int which, int32_t* __restrict__ goff, int32_t* __restrict__ gmap,
                               float** __restrict__ gc) {
    const uint32_t epoch = *e.epoch;
    const EpCtrl* c = ctrl_of(e, e.rank);
    const uint32_t* flags = which == 0 ? c->flag_dispatch : which == 1 ? c->flag_return : c->flag_gather;
    if ((int)threadIdx.x < e.world) {
        bool ok = false;
        for (uint32_t it = 0; it < e.spin_limit; ++it) {
            if ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - epoch) >= 0) { ok = true; break; }
            __nanosleep(100);
        }
        if (!ok) atomicExch(e.status, 1);
    }
    __syncthreads();
    if (goff && threadIdx.x == 0) {
        int g = 0;
        for (int s = 0; s < e.world; ++s) {
            const int32_t* h = hdr_of(e, e.rank, s);
            int at = s * e.cap;
            const int end = (s + 1) * e.cap;
            // row (s cap + j) of the receive buffer is row (base + j) of sender s's order
            float* const home = reinterpret_cast<float*>(e.peers[s] + e.off_y) + ((int64_t)h[e.nl] - (int64_t)s * e.cap) * e.d;
            for (int x = 0; x < e.nl; ++x, ++g) {
                goff[g] = at;
                gmap[g] = x;
                gc[g] = home;
                at = min(at + max(h[x], 0), end);
            }
            goff[g] = at;
            gmap[g] = -1;
            gc[g] = home;
            ++g;
        }
        goff[g] = e.world * e.cap;
    }
    if (which == 2 && threadIdx.x == 0) *e.epoch = epoch + 1;       // the pass is complete on this rank
}

// The down projection stored its result rows straight into the senders' y buffers (per-group
// output bases); all of that kernel's stores are complete when this one starts, so one
// thread fences and tells every sender that its results are home.
__global__ void ep_returned_kernel(EpDev e) {
    const uint32_t epoch = *e.epoch;
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < e.world; ++r) st_release_sys(&ctrl_of(e, r)->flag_return[e.rank], epoch);
    }
}

// The combination of my slice stored straight into every rank's output:
// out[lo + t, :] = (shared ? part[t, :] : 0) + sum_k w[t, k] * y[inv[t K + k], :], k ascending
// (the arithmetic of the single-GPU layer's combination, separate multiply and add).
__global__ void __launch_bounds__(256) ep_combine_gather_kernel(EpDev e, const float* __restrict__ y,
                                                                const int32_t* __restrict__ inv, const float* __restrict__ w,
                                                                const float* __restrict__ part, int n, int K, int64_t lo,
                                                                int has_shared) {
    const uint32_t epoch = *e.epoch;
    const int d4 = e.d >> 2;
    const int64_t total = (int64_t)n * d4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / d4), j = (int)(i - (int64_t)t * d4);
        float4 acc = has_shared ? *(reinterpret_cast<const float4*>(part + (int64_t)t * e.d) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < K; ++k) {
            const int slot = t * K + k;
            const float wk = w[slot];
            const float4 v = *(reinterpret_cast<const float4*>(y + (int64_t)inv[slot] * e.d) + j);
            acc.x = __fadd_rn(acc.x, __fmul_rn(wk, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(wk, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(wk, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(wk, v.w));
        }
        for (int r = 0; r < e.world; ++r)
            *(reinterpret_cast<float4*>(e.peers[r] + e.off_out) + (lo + t) * d4 + j) = acc;
    }
    if (grid_last_cta(&ctrl_of(e, e.rank)->done[2]))
        for (int q = 0; q < e.world; ++q) st_release_sys(&ctrl_of(e, q)->flag_gather[e.rank], epoch);
}

}  // namespace b200

using namespace b200;

struct b200_ep {
    int rank = 0, world = 1, d = 0, E = 0, ne = 0, K = 0, SH = 0, qkind = 0, nl = 0;
    int max_T = 0, slice_max = 0, cap = 0;
    size_t off_hdr = 0, off_rows = 0, off_y = 0, off_out = 0, block_bytes = 0;
    char* block = nullptr;                       // my symmetric block
    char* peer[EP_MAXW] = {};                    // mapped peers (peer[rank] == block)
    bool opened[EP_MAXW] = {};                   // mapped through CUDA IPC (to be closed)
    char** peers_dev = nullptr;
    bool connected = false;
    // local buffers
    int32_t *idx = nullptr, *inv = nullptr, *offsets = nullptr, *goff = nullptr, *gmap = nullptr;
    float *w = nullptr, *part = nullptr;
    float** gc = nullptr;                        // per GEMM group: where its result rows go (peer memory)
    void* sh_scratch = nullptr;                  // the shared expert's own scratch: it runs on a second stream
    int32_t* grouped = nullptr;
    // weights
    const float *router_w = nullptr, *router_bias = nullptr;
    const void *gates = nullptr, *ups = nullptr, *downs = nullptr, *sh_g = nullptr, *sh_u = nullptr, *sh_d = nullptr;
    uint32_t* epoch_dev = nullptr;               // number of the pass in flight (starts at 1)
    bool begun = false;                          // phase 0 has run at least once
    uint32_t spin_limit = EP_SPIN_DEFAULT;
    // b200_ep_forward replays a recording of the pass when called again with the same x and T
    cudaGraphExec_t graph = nullptr;
    const float* graph_x = nullptr;
    int graph_T = 0, eager_passes = 0;
    unsigned long long graph_ws_generation = 0;
    cudaStream_t own_stream = nullptr;
    int T = 0, lo = 0, n = 0;                    // the pass in flight
    bool shared_pending = false;                 // the shared expert of this pass runs on the second stream
};

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
static void slice_of(int T, int rank, int world, int* lo, int* hi) {
    *lo = (int)((int64_t)rank * T / world);
    *hi = (int)((int64_t)(rank + 1) * T / world);
}

static EpDev dev_args(const b200_ep* ep) {
    EpDev e;
    e.rank = ep->rank; e.world = ep->world; e.nl = ep->nl; e.cap = ep->cap; e.d = ep->d;
    e.peers = ep->peers_dev;
    e.off_hdr = ep->off_hdr; e.off_rows = ep->off_rows; e.off_y = ep->off_y; e.off_out = ep->off_out;
    e.status = stream_status_ptr();
    e.spin_limit = ep->spin_limit;
    e.epoch = ep->epoch_dev;
    return e;
}

static int upload_peers(b200_ep* ep) {
    B200_CUDA(cudaMemcpy(ep->peers_dev, ep->peer, sizeof(char*) * ep->world, cudaMemcpyHostToDevice));
    ep->connected = true;
    return B200_OK;
}

extern "C" {

int b200_ep_create(b200_ep** out, int rank, int world, int d, int E, int ne, int K, int SH, int qkind, int max_tokens,
                   int capacity_rows) {
    B200_REQUIRE(out, "ep_create: null pointer");
    B200_REQUIRE(world >= 1 && world <= EP_MAXW && rank >= 0 && rank < world, "ep_create: rank %d of %d", rank, world);
    B200_REQUIRE(ne >= 1 && ne % world == 0, "ep_create: %d experts do not divide over %d ranks", ne, world);
    B200_REQUIRE(d >= 32 && d % 32 == 0 && E % 32 == 0 && K >= 1 && K <= ne && max_tokens >= 1 && SH >= 0,
                 "ep_create: bad sizes");
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "ep_create: unknown qkind %d", qkind);
    B200_REQUIRE(stream_status_ptr() != nullptr, "ep_create: no status word");
    B200_REQUIRE(((int64_t)(max_tokens + world - 1) / world) * K * world <= 0x7fffffff, "ep_create: too many rows");
    b200_ep* ep = new b200_ep();
    ep->rank = rank; ep->world = world; ep->d = d; ep->E = E; ep->ne = ne; ep->K = K; ep->SH = SH; ep->qkind = qkind;
    ep->nl = ne / world;
    ep->max_T = max_tokens;
    ep->slice_max = (max_tokens + world - 1) / world;
    const int64_t worst = (int64_t)ep->slice_max * K;
    ep->cap = capacity_rows > 0 ? (int)std::min<int64_t>(capacity_rows, worst) : (int)worst;
    ep->off_hdr = sizeof(EpCtrl);
    ep->off_rows = up256(ep->off_hdr + (size_t)world * (ep->nl + 2) * 4);
    ep->off_y = up256(ep->off_rows + (size_t)world * ep->cap * d * 2);
    ep->off_out = up256(ep->off_y + (size_t)worst * d * 4);
    ep->block_bytes = up256(ep->off_out + (size_t)max_tokens * d * 4);
    auto fail_free = [&](int rc) {
        b200_ep_destroy(ep);
        return rc;
    };
    auto alloc = [&](void** p, size_t bytes) -> int {
        B200_CUDA(cudaMalloc(p, std::max<size_t>(bytes, 256)));
        B200_CUDA(cudaMemset(*p, 0, std::max<size_t>(bytes, 256)));
        return B200_OK;
    };
    int rc = alloc(reinterpret_cast<void**>(&ep->block), ep->block_bytes);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->peers_dev), sizeof(char*) * EP_MAXW);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->idx), (size_t)worst * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->w), (size_t)worst * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->inv), (size_t)worst * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->grouped), (size_t)worst * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->offsets), (size_t)(ne + 1) * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->goff), (size_t)(world * (ep->nl + 1) + 1) * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->gmap), (size_t)(world * (ep->nl + 1)) * 4);
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->gc), (size_t)(world * (ep->nl + 1)) * sizeof(float*));
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->part), (size_t)ep->slice_max * d * 4);
    if (!rc && SH > 0) rc = alloc(&ep->sh_scratch, moe_shared_scratch_bytes(ep->slice_max, d, SH));
    if (!rc) rc = alloc(reinterpret_cast<void**>(&ep->epoch_dev), 256);
    if (!rc) {
        const uint32_t one = 1;
        const cudaError_t e = cudaMemcpy(ep->epoch_dev, &one, 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) rc = cuda_status(e, "ep_create: pass counter");
    }
    if (rc) return fail_free(rc);
    ep->peer[rank] = ep->block;
    if (world == 1) {
        rc = upload_peers(ep);
        if (rc) return fail_free(rc);
    }
    *out = ep;
    return B200_OK;
}

int b200_ep_destroy(b200_ep* ep) {
    if (!ep) return B200_OK;
    cudaDeviceSynchronize();
    if (ep->graph) cudaGraphExecDestroy(ep->graph);
    if (ep->own_stream) cudaStreamDestroy(ep->own_stream);
    for (int r = 0; r < ep->world; ++r)
        if (ep->opened[r] && ep->peer[r]) cudaIpcCloseMemHandle(ep->peer[r]);
    for (void* p : {(void*)ep->block, (void*)ep->peers_dev, (void*)ep->idx, (void*)ep->w, (void*)ep->inv, (void*)ep->grouped,
                    (void*)ep->offsets, (void*)ep->goff, (void*)ep->gmap, (void*)ep->gc, (void*)ep->part, ep->sh_scratch, (void*)ep->epoch_dev})
        if (p) cudaFree(p);
    delete ep;
    return B200_OK;
}

int b200_ep_set_weights(b200_ep* ep, const float* router_w, const float* router_bias, const void* gates_local,
                        const void* ups_local, const void* downs_local, const void* sh_gate, const void* sh_up,
                        const void* sh_down) {
    B200_REQUIRE(ep && router_w && gates_local && ups_local && downs_local, "ep_set_weights: null pointer");
    ep->router_w = router_w; ep->router_bias = router_bias;
    ep->gates = gates_local; ep->ups = ups_local; ep->downs = downs_local;
    ep->sh_g = sh_gate; ep->sh_u = sh_up; ep->sh_d = sh_down;
    return B200_OK;
}

int b200_ep_export(b200_ep* ep, void* handle_out) {
    B200_REQUIRE(ep && handle_out, "ep_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == B200_EP_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    B200_CUDA(cudaIpcGetMemHandle(&h, ep->block));
    memcpy(handle_out, &h, sizeof(h));
    return B200_OK;
}

int b200_ep_connect(b200_ep* ep, const void* handles_all) {
    B200_REQUIRE(ep && handles_all, "ep_connect: null pointer");
    B200_REQUIRE(!ep->connected || ep->world == 1, "ep_connect: already connected");
    for (int r = 0; r < ep->world; ++r) {
        if (r == ep->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles_all) + (size_t)r * B200_EP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        B200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ep->peer[r] = static_cast<char*>(p);
        ep->opened[r] = true;
    }
    return upload_peers(ep);
}

int b200_ep_connect_local(b200_ep* ep, b200_ep* const* peers) {
    B200_REQUIRE(ep && peers, "ep_connect_local: null pointer");
    int mine = 0;
    B200_CUDA(cudaGetDevice(&mine));
    for (int r = 0; r < ep->world; ++r) {
        B200_REQUIRE(peers[r] && peers[r]->rank == r && peers[r]->world == ep->world && peers[r]->block_bytes == ep->block_bytes,
                     "ep_connect_local: peer %d does not match", r);
        ep->peer[r] = peers[r]->block;
        cudaPointerAttributes at;
        B200_CUDA(cudaPointerGetAttributes(&at, peers[r]->block));
        if (at.device != mine) {
            const cudaError_t e = cudaDeviceEnablePeerAccess(at.device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_status(e, "ep_connect_local: peer access");
            cudaGetLastError();
        }
    }
    return upload_peers(ep);
}

int b200_ep_rendezvous_dir(b200_ep* ep, const char* dir, int timeout_ms) {
    B200_REQUIRE(ep && dir, "ep_rendezvous_dir: null pointer");
    if (ep->world == 1) return B200_OK;
    char mine[B200_EP_HANDLE_BYTES];
    int rc = b200_ep_export(ep, mine);
    if (rc) return rc;
    auto path_of = [&](int r) { return std::string(dir) + "/b200ep." + std::to_string(r); };
    {
        const std::string tmp = path_of(ep->rank) + ".tmp";
        FILE* f = fopen(tmp.c_str(), "wb");
        B200_REQUIRE(f, "ep_rendezvous_dir: cannot write %s", tmp.c_str());
        const size_t n = fwrite(mine, 1, sizeof(mine), f);
        fclose(f);
        B200_REQUIRE(n == sizeof(mine) && rename(tmp.c_str(), path_of(ep->rank).c_str()) == 0,
                     "ep_rendezvous_dir: cannot publish %s", path_of(ep->rank).c_str());
    }
    std::vector<char> all((size_t)ep->world * B200_EP_HANDLE_BYTES);
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < ep->world; ++r) {
        for (;;) {
            FILE* f = fopen(path_of(r).c_str(), "rb");
            if (f) {
                const size_t n = fread(all.data() + (size_t)r * B200_EP_HANDLE_BYTES, 1, B200_EP_HANDLE_BYTES, f);
                fclose(f);
                if (n == B200_EP_HANDLE_BYTES) break;
            }
            const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            B200_REQUIRE(ms < timeout_ms, "ep_rendezvous_dir: rank %d did not appear in %s within %d ms", r, dir, timeout_ms);
            std::this_thread::sleep_for(std::chrono::milliseconds(5));
        }
    }
    return b200_ep_connect(ep, all.data());
}

int b200_ep_phase(b200_ep* ep, int phase, const float* x, int T) {
    B200_REQUIRE(ep && ep->connected, "ep_phase: not connected");
    B200_REQUIRE(ep->gates, "ep_phase: no weights set");
    B200_REQUIRE(phase >= 0 && phase <= 3, "ep_phase: phase %d", phase);
    static const char* const names[4] = {"b200.ep.route+dispatch", "b200.ep.experts+return", "b200.ep.combine+gather",
                                         "b200.ep.wait_slices"};
    NvtxRange range(names[phase]);
    cudaStream_t st = stream();
    const int d = ep->d, K = ep->K, G = ep->world;
    int rc;
    if (phase == 0) {
        B200_REQUIRE(x && T >= 1 && T <= ep->max_T, "ep_phase: T = %d outside 1 .. %d", T, ep->max_T);
        int lo, hi;
        slice_of(T, ep->rank, G, &lo, &hi);
        ep->T = T; ep->lo = lo; ep->n = hi - lo;
        ep->begun = true;
        const int n = ep->n;
        const float* xs = x + (int64_t)lo * d;
        // the shared expert of my own tokens: on the second stream, next to everything up to
        // the combination (its scratch is the handle's own)
        ep->shared_pending = false;
        if (n > 0 && ep->sh_g && ep->sh_u && ep->sh_d && ep->SH > 0) {
            rc = side_begin();
            if (rc) return rc;
            rc = moe_shared_expert(xs, ep->sh_g, ep->sh_u, ep->sh_d, ep->part, n, d, ep->SH, tag_of_qkind(ep->qkind),
                                   ep->sh_scratch);
            const int rc2 = side_end();
            if (rc || rc2) return rc ? rc : rc2;
            ep->shared_pending = true;
        }
        if (n > 0) {
            rc = b200_moe_route(xs, ep->router_w, ep->router_bias, nullptr, ep->idx, ep->w, n, d, ep->ne, K);
            if (rc) return rc;
            rc = moe_dispatch_perm(ep->idx, n, ep->ne, K, ep->grouped, ep->inv, ep->offsets);
            if (rc) return rc;
        } else {
            B200_CUDA(cudaMemsetAsync(ep->offsets, 0, (size_t)(ep->ne + 1) * 4, st));
        }
        const int64_t NK = (int64_t)n * K;
        const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div64(NK, 8), (int64_t)num_sms() * 8));
        ep_pack_dispatch_kernel<<<grid, 256, 0, st>>>(dev_args(ep), xs, ep->grouped, K, ep->offsets, NK);
        B200_LAUNCH_CHECK("ep_pack_dispatch_kernel");
        return B200_OK;
    }
    B200_REQUIRE(ep->begun, "ep_phase: phase %d before phase 0", phase);
    if (phase == 1) {
        ep_wait_kernel<<<1, 32, 0, st>>>(dev_args(ep), 0, ep->goff, ep->gmap, ep->gc);
        B200_LAUNCH_CHECK("ep_wait_kernel");
        const int groups = G * (ep->nl + 1);
        rc = moe_experts_rows(reinterpret_cast<const __half*>(ep->block + ep->off_rows), ep->goff, ep->gmap, groups,
                              (int64_t)G * ep->cap, ep->gates, ep->ups, ep->downs, ep->nl, nullptr, d, ep->E,
                              tag_of_qkind(ep->qkind), ep->gc);
        if (rc) return rc;
        ep_returned_kernel<<<1, 32, 0, st>>>(dev_args(ep));
        B200_LAUNCH_CHECK("ep_returned_kernel");
        return B200_OK;
    }
    if (phase == 2) {
        ep_wait_kernel<<<1, 32, 0, st>>>(dev_args(ep), 1, nullptr, nullptr, nullptr);
        B200_LAUNCH_CHECK("ep_wait_kernel");
        const bool shared = ep->shared_pending;
        if (shared && (rc = side_wait())) return rc;
        ep->shared_pending = false;
        const int64_t vecs = (int64_t)ep->n * (d >> 2);
        const int gx = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div64(vecs, 256), (int64_t)num_sms() * 16));
        ep_combine_gather_kernel<<<gx, 256, 0, st>>>(dev_args(ep), reinterpret_cast<const float*>(ep->block + ep->off_y), ep->inv,
                                                     ep->w, ep->part, ep->n, K, ep->lo, shared ? 1 : 0);
        B200_LAUNCH_CHECK("ep_combine_gather_kernel");
        return B200_OK;
    }
    ep_wait_kernel<<<1, 32, 0, st>>>(dev_args(ep), 2, nullptr, nullptr, nullptr);
    B200_LAUNCH_CHECK("ep_wait_kernel");
    return B200_OK;
}

static int forward_eager(b200_ep* ep, const float* x, int T) {
    for (int phase = 0; phase < 4; ++phase) {
        const int rc = b200_ep_phase(ep, phase, x, T);
        if (rc) return rc;
    }
    return B200_OK;
}

// The first two passes with a given (x, T) run eagerly (they size the library's workspaces);
// the third is recorded into a CUDA graph - the pass reads nothing on the host, its number
// lives in device memory - and later ones replay it as one launch.  A recording is dropped
// when one of the library's workspaces has moved since.
int b200_ep_forward(b200_ep* ep, const float* x, int T) {
    B200_REQUIRE(ep && ep->connected, "ep_forward: not connected");
    if (ep->graph && (ep->graph_x != x || ep->graph_T != T || ep->graph_ws_generation != workspace_generation())) {
        cudaGraphExecDestroy(ep->graph);
        ep->graph = nullptr;
        ep->eager_passes = 0;
    }
    if (!ep->graph) {
        if (ep->graph_x != x || ep->graph_T != T) {
            ep->graph_x = x;
            ep->graph_T = T;
            ep->eager_passes = 0;
        }
        if (ep->eager_passes < 2) {
            ep->eager_passes += 1;
            return forward_eager(ep, x, T);
        }
        if (!ep->own_stream) B200_CUDA(cudaStreamCreateWithFlags(&ep->own_stream, cudaStreamNonBlocking));
        cudaStream_t prev = stream();
        // the recording starts after everything enqueued so far
        cudaEvent_t ev;
        B200_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        cudaEventRecord(ev, prev);
        cudaStreamWaitEvent(ep->own_stream, ev, 0);
        cudaEventDestroy(ev);
        b200_set_stream(ep->own_stream);
        cudaGraph_t g = nullptr;
        int rc = B200_OK;
        cudaError_t e = cudaStreamBeginCapture(ep->own_stream, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            rc = forward_eager(ep, x, T);
            e = cudaStreamEndCapture(ep->own_stream, &g);
        }
        b200_set_stream(prev);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) return cuda_status(e, "ep_forward: stream capture");
        e = cudaGraphInstantiate(&ep->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return cuda_status(e, "ep_forward: cudaGraphInstantiate");
        ep->graph_ws_generation = workspace_generation();
    }
    B200_CUDA(cudaGraphLaunch(ep->graph, stream()));
    return B200_OK;
}

int b200_ep_output(b200_ep* ep, const float** out_dev) {
    B200_REQUIRE(ep && out_dev, "ep_output: null pointer");
    *out_dev = reinterpret_cast<const float*>(ep->block + ep->off_out);
    return B200_OK;
}

int b200_ep_routing(b200_ep* ep, const int32_t** idx_dev, const float** w_dev, int* n_slice) {
    B200_REQUIRE(ep, "ep_routing: null handle");
    if (idx_dev) *idx_dev = ep->idx;
    if (w_dev) *w_dev = ep->w;
    if (n_slice) *n_slice = ep->n;
    return B200_OK;
}

int b200_ep_set_spin_limit(b200_ep* ep, int spin_limit) {
    B200_REQUIRE(ep && spin_limit >= 0, "ep_set_spin_limit: bad arguments");
    ep->spin_limit = spin_limit > 0 ? (uint32_t)spin_limit : EP_SPIN_DEFAULT;
    return B200_OK;
}

int b200_ep_link_bytes(b200_ep* ep, double* bytes) {
    B200_REQUIRE(ep && bytes, "ep_link_bytes: null pointer");
    std::vector<int32_t> off((size_t)ep->ne + 1);
    B200_CUDA(cudaMemcpyAsync(off.data(), ep->offsets, off.size() * 4, cudaMemcpyDeviceToHost, stream()));
    B200_CUDA(cudaStreamSynchronize(stream()));
    const int64_t mine = off[(size_t)(ep->rank + 1) * ep->nl] - off[(size_t)ep->rank * ep->nl];
    const int64_t away = (int64_t)ep->n * ep->K - mine;                     // rows that left this GPU
    // rows out in fp16; the same number of result rows comes back in fp32 from the expert ranks
    // (counted where they are sent: by symmetry of the pass, on average, the same amount);
    // the output slice goes to world - 1 peers
    *bytes = (double)away * ep->d * 2 + (double)away * ep->d * 4 + (double)(ep->world - 1) * ep->n * ep->d * 4;
    return B200_OK;
}

}  // extern "C"
