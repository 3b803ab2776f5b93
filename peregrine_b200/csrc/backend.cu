// Host side of libcoli_cuda_backend.so: contexts, residency, the expert-group
// calls of the reference ABI and the device-resident MoE layer.  Declarations
// and the reference lines each entry point replaces are in
// include/peregrine_b200.h.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/peregrine_b200.h"
#include "kernels.cuh"
#include "kernels_mma.cuh"
#include "kernels_tile.cuh"
#include "kernels_umma.cuh"
#include "kernels_block.cuh"
#include "kernels_decode.cuh"
#include "kernels_ep.cuh"
#include "w4_host.h"

using namespace pgb;

#define PGB_EXPORT extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------- contexts
struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
    bool pinned = false;
};

struct Ctx {
    int device = -1;
    cudaStream_t stream = nullptr;
    cudaStream_t side = nullptr;  // runs the exact router chains beside the speculative expert launches
    int sms = 0;
    size_t smem_optin = 0;
    size_t tensor_count = 0, tensor_bytes = 0;
    int *err_dev = nullptr;
    uint64_t scratch_gen = 0;
    // expert-group scratch (grow-only, per device; one caller thread per device)
    DevBuf x, y, h, xq, sx, xcs, hq, sh, hcs, slots_gu, slots_dn, slots_f32, nslots, csr_ptr, csr_idx, csr_rw, out;
    DevBuf pin_x, pin_y, pin_slots;
    DevBuf pipe[24];
    bool capturing = false;
    // Shape cache of the expert-group call (COLI_CUDA_GRAPH=1), bookkeeping only: which launch
    // shapes have been seen under which scratch generation (cuda/backend_cuda.cu:678-745).
    struct ShapeSlot {
        uint64_t key = 0, gen = 0, used = 0;
    } shapes[16];
    uint64_t shape_clock = 0;
};

static Ctx g_ctx[COLI_CUDA_MAX_DEVICES];
static int g_nctx = 0;
static std::mutex g_stats_mu;
static uint64_t g_calls = 0, g_experts = 0, g_rows = 0;
static double g_h2d_ms = 0, g_kernel_ms = 0, g_d2h_ms = 0;
static uint64_t g_captures = 0, g_replays = 0, g_invalidations = 0, g_uncacheable = 0;
static std::atomic<uint64_t> g_launches{0};

static int cuda_ok(cudaError_t err, const char *what) {
    if (err == cudaSuccess) return 1;
    std::fprintf(stderr, "[CUDA] %s: %s\n", what, cudaGetErrorString(err));
    return 0;
}
static int fail(const char *what) {
    std::fprintf(stderr, "[CUDA] %s\n", what);
    return 0;
}

static Ctx *find_ctx(int device) {
    for (int i = 0; i < g_nctx; ++i)
        if (g_ctx[i].device == device) return &g_ctx[i];
    return nullptr;
}

static thread_local int t_current_device = -1;
static int select_ctx(Ctx *c) {
    if (!c) return 0;
    if (t_current_device == c->device) return 1;
    if (!cuda_ok(cudaSetDevice(c->device), "select device")) return 0;
    t_current_device = c->device;
    return 1;
}

static int env_flag(const char *name, int dflt) {
    const char *v = std::getenv(name);
    return v ? std::atoi(v) : dflt;
}

static void free_buf(DevBuf &b) {
    if (b.p) {
        if (b.pinned)
            cudaFreeHost(b.p);
        else
            cudaFree(b.p);
    }
    b.p = nullptr;
    b.cap = 0;
}

// grow-only reservation; a growth waits for the stream so no kernel still reads the old block
static int reserve(Ctx *c, DevBuf &b, size_t bytes, bool pinned = false) {
    if (bytes <= b.cap && b.p) return 1;
    if (bytes == 0) bytes = 16;
    if (b.p) {
        if (!cuda_ok(cudaStreamSynchronize(c->stream), "scratch growth sync")) return 0;
        free_buf(b);
        c->scratch_gen++;
    }
    b.pinned = pinned;
    const size_t want = (bytes + 255) & ~(size_t)255;
    cudaError_t e = pinned ? cudaMallocHost(&b.p, want) : cudaMalloc(&b.p, want);
    if (!cuda_ok(e, pinned ? "pinned scratch allocation" : "scratch allocation")) {
        b.p = nullptr;
        return 0;
    }
    b.cap = want;
    return 1;
}

// Launch that may begin while the previous launch of the stream is still running (programmatic
// dependent launch); the kernel orders itself with griddepcontrol.wait.
template <typename... KArgs, typename... Args>
static int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      const char *what, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_ok(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...), what);
}

template <typename... KArgs, typename... Args>
static int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const char *what,
                  Args... args) {
    kernel<<<grid, block, smem, stream>>>(args...);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_ok(cudaGetLastError(), what);
}

// Dynamic shared-memory opt-in per kernel.  cudaFuncSetAttribute applies to the current device
// only, so the record of what has been set is kept per context slot (cleared at shutdown): the
// attribute is (re)set whenever a launch on that device needs more than was recorded for it.
struct SmemOptIn {
    const void *fn;
    int bytes;
};
static std::vector<SmemOptIn> g_smem_optin[COLI_CUDA_MAX_DEVICES];
static std::mutex g_smem_mu;

template <typename K>
static int ensure_smem(Ctx *c, K kernel, size_t bytes, const char *what) {
    if (bytes <= 48 * 1024) return 1;
    const void *fn = reinterpret_cast<const void *>(kernel);
    std::lock_guard<std::mutex> lk(g_smem_mu);
    std::vector<SmemOptIn> &tab = g_smem_optin[c - g_ctx];
    for (SmemOptIn &e : tab)
        if (e.fn == fn) {
            if (e.bytes >= (int)bytes) return 1;
            if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what))
                return 0;
            e.bytes = (int)bytes;
            return 1;
        }
    if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what)) return 0;
    tab.push_back({fn, (int)bytes});
    return 1;
}

PGB_EXPORT int coli_cuda_probe_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

PGB_EXPORT void coli_cuda_shutdown(void);

// The side stream carries the exact router chains, which the down launch waits for: highest
// priority, so its few CTAs are placed before the expert launches that run beside them.
static cudaError_t create_side_stream(cudaStream_t *st) {
    int lo = 0, hi = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (e != cudaSuccess) return e;
    return cudaStreamCreateWithPriority(st, cudaStreamNonBlocking, hi);
}

PGB_EXPORT int coli_cuda_init(const int *devices, int count) {
    int available = 0;
    if (!devices || count < 1 || count > COLI_CUDA_MAX_DEVICES) return 0;
    if (!cuda_ok(cudaGetDeviceCount(&available), "device discovery")) return 0;
    if (g_nctx) coli_cuda_shutdown();
    for (int i = 0; i < count; ++i) {
        const int device = devices[i];
        if (device < 0 || device >= available) {
            std::fprintf(stderr, "[CUDA] invalid device %d (available: 0..%d)\n", device, available - 1);
            coli_cuda_shutdown();
            return 0;
        }
        if (find_ctx(device)) {
            std::fprintf(stderr, "[CUDA] duplicate device %d\n", device);
            coli_cuda_shutdown();
            return 0;
        }
        Ctx *c = &g_ctx[g_nctx];
        *c = Ctx();
        c->device = device;
        t_current_device = -1;
        cudaDeviceProp prop{};
        if (!select_ctx(c) || !cuda_ok(cudaGetDeviceProperties(&prop, device), "device properties") ||
            !cuda_ok(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "stream creation") ||
            !cuda_ok(create_side_stream(&c->side), "stream creation") ||
            !cuda_ok(cudaHostAlloc((void **)&c->err_dev, 256, cudaHostAllocMapped | cudaHostAllocPortable),
                     "error word allocation")) {
            g_nctx++;
            coli_cuda_shutdown();
            return 0;
        }
        std::memset(c->err_dev, 0, 256);
        c->sms = prop.multiProcessorCount;
        c->smem_optin = prop.sharedMemPerBlockOptin;
        g_nctx++;
        if (prop.major != 10)
            std::fprintf(stderr, "[CUDA] device %d is sm_%d%d: this backend carries sm_100a code only\n", device,
                         prop.major, prop.minor);
        std::fprintf(stderr, "[CUDA] device %d: %s, %.1f GB VRAM, sm_%d%d, %d SMs\n", device, prop.name,
                     prop.totalGlobalMem / 1e9, prop.major, prop.minor, prop.multiProcessorCount);
    }
    return 1;
}

PGB_EXPORT void coli_cuda_shutdown(void) {
    for (int i = 0; i < g_nctx; ++i) {
        Ctx *c = &g_ctx[i];
        t_current_device = -1;
        if (!select_ctx(c)) continue;
        if (c->stream) cudaStreamSynchronize(c->stream);
        DevBuf *bufs[] = {&c->x,        &c->y,        &c->h,         &c->xq,     &c->sx,      &c->xcs,
                          &c->hq,       &c->sh,       &c->hcs,       &c->slots_gu, &c->slots_dn, &c->slots_f32,
                          &c->nslots,   &c->csr_ptr,  &c->csr_idx,   &c->csr_rw, &c->out,     &c->pin_x,
                          &c->pin_y,    &c->pin_slots};
        for (DevBuf *b : bufs) free_buf(*b);
        for (DevBuf &b : c->pipe) free_buf(b);
        if (c->err_dev) cudaFreeHost(c->err_dev);
        if (c->side) cudaStreamDestroy(c->side);
        if (c->stream) cudaStreamDestroy(c->stream);
        *c = Ctx();
        std::lock_guard<std::mutex> lk(g_smem_mu);
        g_smem_optin[i].clear();
    }
    g_nctx = 0;
    t_current_device = -1;
}

PGB_EXPORT int coli_cuda_device_count(void) { return g_nctx; }
PGB_EXPORT int coli_cuda_device_at(int index) { return (index >= 0 && index < g_nctx) ? g_ctx[index].device : -1; }

PGB_EXPORT int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes) {
    Ctx *c = find_ctx(device);
    if (!free_bytes || !total_bytes || !select_ctx(c)) return 0;
    return cuda_ok(cudaMemGetInfo(free_bytes, total_bytes), "memory query");
}

PGB_EXPORT void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes) {
    size_t n = 0, b = 0;
    for (int i = 0; i < g_nctx; ++i)
        if (device < 0 || g_ctx[i].device == device) {
            n += g_ctx[i].tensor_count;
            b += g_ctx[i].tensor_bytes;
        }
    if (tensor_count) *tensor_count = n;
    if (tensor_bytes) *tensor_bytes = b;
}

PGB_EXPORT void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows, double *h2d_ms,
                                      double *kernel_ms, double *d2h_ms) {
    std::lock_guard<std::mutex> lk(g_stats_mu);
    if (calls) *calls = g_calls;
    if (experts) *experts = g_experts;
    if (rows) *rows = g_rows;
    if (h2d_ms) *h2d_ms = g_h2d_ms;
    if (kernel_ms) *kernel_ms = g_kernel_ms;
    if (d2h_ms) *d2h_ms = g_d2h_ms;
}

PGB_EXPORT void coli_cuda_graph_cache_stats(uint64_t *captures, uint64_t *replays, uint64_t *invalidations,
                                            uint64_t *uncacheable) {
    std::lock_guard<std::mutex> lk(g_stats_mu);
    if (captures) *captures = g_captures;
    if (replays) *replays = g_replays;
    if (invalidations) *invalidations = g_invalidations;
    if (uncacheable) *uncacheable = g_uncacheable;
}

PGB_EXPORT int coli_cuda_last_device_error(int device) {
    Ctx *c = find_ctx(device);
    if (!select_ctx(c)) return -1;
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "error word sync")) return -1;
    const int v = *static_cast<volatile int *>(c->err_dev);
    if (v) *static_cast<volatile int *>(c->err_dev) = 0;
    return v;
}
PGB_EXPORT int coli_cuda_selftest_bounded_wait(int device, long long limit_cycles) {
    Ctx *c = find_ctx(device);
    if (!select_ctx(c) || limit_cycles < 1 || limit_cycles > 2000000000LL) return 0;
    return launch(selftest_bounded_wait_kernel, dim3(1), dim3(32), 0, c->stream, "bounded-wait self-test launch",
                  limit_cycles, c->err_dev) &&
           cuda_ok(cudaStreamSynchronize(c->stream), "bounded-wait self-test synchronise");
}
PGB_EXPORT uint64_t coli_cuda_kernel_launches(void) { return g_launches.load(); }
PGB_EXPORT void *coli_cuda_stream(int device) {
    Ctx *c = find_ctx(device);
    return c ? (void *)c->stream : nullptr;
}

// ---------------------------------------------------------------- residency
// fmt as the caller named it (0, 1, 2, 3, 4); storage is one of:
//   kind 0: fp32 [O, I]   (fmt 0, and fmt 1 / fmt 3 expanded on the host at upload)
//   kind 1: int4 tile stream, per-row scales   (fmt 2)
//   kind 2: int4 tile stream, group scales     (fmt 4)
struct ColiCudaTensor {
    int fmt, I, O, device, kind, gs;
    W4Layout L;
    void *data;         // fp32 matrix or tile stream
    float *row_scales;  // kind 1: padded to ntile*16
    size_t bytes;
};

static size_t src_row_bytes(int fmt, int I) {
    switch (fmt) {
        case 0: return (size_t)I * 4;
        case 1: return (size_t)I;
        case 2:
        case 4: return (size_t)(I + 1) / 2;
        case 3: return (size_t)(I + 3) / 4;
    }
    return 0;
}

// Fills the tensor's device storage from caller-format host data.
static int tensor_fill(Ctx *c, ColiCudaTensor *t, const void *weights, const float *scales) {
    if (t->kind == 0) {
        const size_t n = (size_t)t->O * t->I;
        if (t->fmt == 0) return cuda_ok(cudaMemcpy(t->data, weights, n * 4, cudaMemcpyHostToDevice), "tensor upload");
        // int8 / int2 sources: expand to the fp32 values the reference's generic arm
        // reads (cuda/backend_cuda.cu:101-112) times the row scale.
        std::vector<float> f(n);
        const uint8_t *q = static_cast<const uint8_t *>(weights);
        const size_t rb = src_row_bytes(t->fmt, t->I);
        for (int o = 0; o < t->O; ++o)
            for (int i = 0; i < t->I; ++i) {
                float v;
                if (t->fmt == 1)
                    v = (float)reinterpret_cast<const int8_t *>(q + o * rb)[i];
                else
                    v = (float)(((q[o * rb + (i >> 2)] >> ((i & 3) * 2)) & 3) - 2);
                f[(size_t)o * t->I + i] = v * scales[o];
            }
        return cuda_ok(cudaMemcpy(t->data, f.data(), n * 4, cudaMemcpyHostToDevice), "tensor upload");
    }
    std::vector<uint8_t> stream(t->L.total_bytes);
    std::vector<float> rs(t->kind == 1 ? (size_t)t->L.ntile * kTileRows : 0);
    w4_repack(t->L, static_cast<const uint8_t *>(weights), scales, stream.data(), rs.empty() ? nullptr : rs.data(), 0);
    if (!cuda_ok(cudaMemcpy(t->data, stream.data(), stream.size(), cudaMemcpyHostToDevice), "tensor upload")) return 0;
    if (t->kind == 1 &&
        !cuda_ok(cudaMemcpy(t->row_scales, rs.data(), rs.size() * 4, cudaMemcpyHostToDevice), "scale upload"))
        return 0;
    (void)c;
    return 1;
}

static int tensor_upload_impl(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt, int I, int O,
                              int gs, int device) {
    Ctx *c = find_ctx(device);
    if (!tensor || !weights || I < 1 || O < 1 || !select_ctx(c)) return 0;
    if (!src_row_bytes(fmt, I) || (fmt && !scales)) return 0;
    if (*tensor) {
        ColiCudaTensor *t = *tensor;
        return t->fmt == fmt && t->I == I && t->O == O && t->device == device && (fmt != 4 || t->gs == gs);
    }
    ColiCudaTensor *t = static_cast<ColiCudaTensor *>(std::calloc(1, sizeof(ColiCudaTensor)));
    if (!t) return 0;
    t->fmt = fmt;
    t->I = I;
    t->O = O;
    t->device = device;
    t->gs = (fmt == 4) ? gs : 0;
    t->kind = (fmt == 2) ? 1 : (fmt == 4) ? 2 : 0;
    if (t->kind) {
        if (!w4_layout_make(&t->L, O, I, t->kind == 2, gs)) {
            std::free(t);
            return fail("int4 upload: group size must be a multiple of 32 and at most 256");
        }
        t->bytes = t->L.total_bytes + (t->kind == 1 ? (size_t)t->L.ntile * kTileRows * 4 : 0);
    } else {
        t->bytes = (size_t)O * I * 4;
    }
    const size_t main_bytes = t->kind ? t->L.total_bytes : t->bytes;
    if (!cuda_ok(cudaMalloc(&t->data, main_bytes), "tensor allocation") ||
        (t->kind == 1 &&
         !cuda_ok(cudaMalloc(&t->row_scales, (size_t)t->L.ntile * kTileRows * 4), "scale allocation")) ||
        !tensor_fill(c, t, weights, scales)) {
        if (t->data) cudaFree(t->data);
        if (t->row_scales) cudaFree(t->row_scales);
        std::free(t);
        return 0;
    }
    c->tensor_count++;
    c->tensor_bytes += t->bytes;
    *tensor = t;
    return 1;
}

PGB_EXPORT int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt,
                                       int I, int O, int device) {
    if (fmt < 0 || fmt > 3) return 0;
    return tensor_upload_impl(tensor, weights, scales, fmt, I, O, 0, device);
}

PGB_EXPORT int coli_cuda_tensor_upload_grouped(ColiCudaTensor **tensor, const void *weights, const float *scales,
                                               int I, int O, int gs, int device) {
    return tensor_upload_impl(tensor, weights, scales, 4, I, O, gs, device);
}

PGB_EXPORT int coli_cuda_tensor_update(ColiCudaTensor *tensor, const void *weights, const float *scales) {
    if (!tensor || !weights || (tensor->fmt && !scales)) return 0;
    Ctx *c = find_ctx(tensor->device);
    if (!select_ctx(c)) return 0;
    // kernels of earlier calls may still read the old contents
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "tensor refresh sync")) return 0;
    return tensor_fill(c, tensor, weights, scales);
}

// A second resident copy of a tensor, made on the device (no host data needed): same format and
// contents, its own memory.
PGB_EXPORT int coli_cuda_tensor_clone(ColiCudaTensor **out, const ColiCudaTensor *src) {
    if (!out || !src || *out) return 0;
    Ctx *c = find_ctx(src->device);
    if (!select_ctx(c)) return 0;
    ColiCudaTensor *t = static_cast<ColiCudaTensor *>(std::calloc(1, sizeof(ColiCudaTensor)));
    if (!t) return 0;
    *t = *src;
    t->data = nullptr;
    t->row_scales = nullptr;
    const size_t main_bytes = t->kind ? t->L.total_bytes : t->bytes;
    const size_t rs_bytes = t->kind == 1 ? (size_t)t->L.ntile * kTileRows * 4 : 0;
    if (!cuda_ok(cudaMalloc(&t->data, main_bytes), "tensor allocation") ||
        (rs_bytes && !cuda_ok(cudaMalloc(&t->row_scales, rs_bytes), "scale allocation")) ||
        !cuda_ok(cudaMemcpy(t->data, src->data, main_bytes, cudaMemcpyDeviceToDevice), "tensor clone") ||
        (rs_bytes && !cuda_ok(cudaMemcpy(t->row_scales, src->row_scales, rs_bytes, cudaMemcpyDeviceToDevice), "scale clone"))) {
        if (t->data) cudaFree(t->data);
        if (t->row_scales) cudaFree(t->row_scales);
        std::free(t);
        return 0;
    }
    c->tensor_count++;
    c->tensor_bytes += t->bytes;
    *out = t;
    return 1;
}

PGB_EXPORT void coli_cuda_tensor_free(ColiCudaTensor *tensor) {
    if (!tensor) return;
    Ctx *c = find_ctx(tensor->device);
    if (select_ctx(c)) {
        cudaStreamSynchronize(c->stream);
        if (tensor->data) cudaFree(tensor->data);
        if (tensor->row_scales) cudaFree(tensor->row_scales);
        if (c->tensor_count) c->tensor_count--;
        c->tensor_bytes = c->tensor_bytes >= tensor->bytes ? c->tensor_bytes - tensor->bytes : 0;
    }
    std::free(tensor);
}
PGB_EXPORT size_t coli_cuda_tensor_bytes(const ColiCudaTensor *tensor) { return tensor ? tensor->bytes : 0; }
PGB_EXPORT int coli_cuda_tensor_device(const ColiCudaTensor *tensor) { return tensor ? tensor->device : -1; }

// ------------------------------------------------------------ GEMV dispatch
static size_t gemv_xs_bytes(int n_xrows, int kp, int nblk) {
    return (((size_t)n_xrows * kp + 15) & ~(size_t)15) + (size_t)n_xrows * nblk * 4 + (size_t)n_xrows * 8 + 16;
}

template <int RMAX, bool GROUPED, int BPG, int XS, bool TAP>
static int gemv_launch_t(Ctx *c, const GemvParams &P, size_t smem) {
    auto kfn = gemv_w4a8_kernel<RMAX, GROUPED, BPG, XS, TAP>;
    if (!ensure_smem(c, kfn, c->smem_optin, "gemv shared-memory opt-in")) return 0;
    if (P.pdl)
        return launch_pdl(kfn, dim3(P.grid > 0 ? P.grid : c->sms), dim3(kGemvThreads), smem, c->stream,
                          "w4a8 gemv launch", P);
    return launch(kfn, dim3(P.grid > 0 ? P.grid : c->sms), dim3(kGemvThreads), smem, c->stream, "w4a8 gemv launch", P);
}

template <int RMAX, bool GROUPED, int BPG>
static int gemv_launch_x(Ctx *c, const GemvParams &P, int xs, size_t smem) {
    // the tap variant is a debugging aid
    if (P.tap) {
        if (xs == 2) return gemv_launch_t<RMAX, GROUPED, BPG, 2, true>(c, P, smem);
        if (xs == 1) return gemv_launch_t<RMAX, GROUPED, BPG, 1, true>(c, P, smem);
        return gemv_launch_t<RMAX, GROUPED, BPG, 0, true>(c, P, smem);
    }
    if (xs == 2) return gemv_launch_t<RMAX, GROUPED, BPG, 2, false>(c, P, smem);
    if (xs == 1) return gemv_launch_t<RMAX, GROUPED, BPG, 1, false>(c, P, smem);
    return gemv_launch_t<RMAX, GROUPED, BPG, 0, false>(c, P, smem);
}

template <int RMAX>
static int gemv_launch_r(Ctx *c, const GemvParams &P, bool grouped, int bpg, int xs, size_t smem) {
    if (!grouped) return gemv_launch_x<RMAX, false, 1>(c, P, xs, smem);
    switch (bpg) {
        case 1: return gemv_launch_x<RMAX, true, 1>(c, P, xs, smem);
        case 2: return gemv_launch_x<RMAX, true, 2>(c, P, xs, smem);
        case 4: return gemv_launch_x<RMAX, true, 4>(c, P, xs, smem);
        case 8: return gemv_launch_x<RMAX, true, 8>(c, P, xs, smem);
    }
    return fail("w4a8 gemv: unsupported group size");
}

// ---- small-batch (tensor-core) variant: 3 or more rows in some slot
template <int NT, bool GROUPED, int BPG, bool TAP>
static int mma_launch_t(Ctx *c, const GemvParams &P) {
    auto kfn = gemv_w4a8_mma_kernel<NT, GROUPED, BPG, TAP>;
    const size_t smem = (size_t)mma_ring_bytes(NT) + kMmaBarBytes;
    if (!ensure_smem(c, kfn, smem, "mma gemv shared-memory opt-in")) return 0;
    return launch(kfn, dim3(c->sms), dim3(kMmaThreads), smem, c->stream, "w4a8 mma gemv launch", P);
}

template <int NT, bool GROUPED, int BPG>
static int mma_launch_x(Ctx *c, const GemvParams &P) {
    return P.tap ? mma_launch_t<NT, GROUPED, BPG, true>(c, P) : mma_launch_t<NT, GROUPED, BPG, false>(c, P);
}

template <int NT>
static int mma_launch_r(Ctx *c, const GemvParams &P, bool grouped, int bpg) {
    if (!grouped) return mma_launch_x<NT, false, 1>(c, P);
    switch (bpg) {
        case 1: return mma_launch_x<NT, true, 1>(c, P);
        case 2: return mma_launch_x<NT, true, 2>(c, P);
        case 4: return mma_launch_x<NT, true, 4>(c, P);
        case 8: return mma_launch_x<NT, true, 8>(c, P);
    }
    return fail("w4a8 mma gemv: unsupported group size");
}

// ---- batched-decode variant: more than 8 rows in some slot; the CTA's warps share the activation rows
template <bool GROUPED, int BPG>
static int block_launch_t(Ctx *c, const GemvParams &P) {
    auto kfn = gemv_w4a8_block_kernel<GROUPED, BPG>;
    if (!ensure_smem(c, kfn, (size_t)kBlkSmemBytes, "block gemv shared-memory opt-in")) return 0;
    return launch(kfn, dim3(c->sms), dim3(kBlkThreads), (size_t)kBlkSmemBytes, c->stream, "w4a8 block gemv launch", P);
}
static int block_launch(Ctx *c, const GemvParams &P0, bool grouped, int bpg) {
    static const int rpp_env = [] {
        const char *e = std::getenv("PEREGRINE_B200_BLOCK_RPP");
        return e ? std::atoi(e) : 0;
    }();
    GemvParams P = P0;
    P.blk_rpp = rpp_env;  // 0: the kernel chooses
    if (!grouped) return block_launch_t<false, 1>(c, P);
    switch (bpg) {
        case 1: return block_launch_t<true, 1>(c, P);
        case 2: return block_launch_t<true, 2>(c, P);
        case 4: return block_launch_t<true, 4>(c, P);
        case 8: return block_launch_t<true, 8>(c, P);
    }
    return fail("w4a8 block gemv: unsupported group size");
}
static int block_min_rows() {
    static const int v = [] {
        const char *e = std::getenv("PEREGRINE_B200_BLOCK_MIN_ROWS");
        return e ? std::atoi(e) : 9;
    }();
    return v;
}

// Rows per expert beyond which the tensor-core kernel (and the chunk-major activation layout) is used.
static bool gemv_uses_mma(int max_rows) { return max_rows > 2; }
// Bytes of the quantised activations of `rows` rows in the layout the kernel for `max_rows` reads.
static size_t act_xq_bytes(const W4Layout &L, size_t rows, int max_rows) {
    return gemv_uses_mma(max_rows) ? (size_t)L.nchunk * rows * kXqChunkRowBytes : rows * (size_t)L.kp;
}

// True when the launch's activation rows fit in shared memory beside the rings of the dp4a kernel.
static bool gemv_rows_fit(Ctx *c, int n_xrows, const W4Layout &L) {
    return (size_t)kRingBytes + kGemvBarBytes + gemv_xs_bytes(n_xrows, L.kp, L.nblk) + 1024 <= c->smem_optin;
}
// True when a down launch with these bounds will quantise its fp32 rows itself.
static bool gemv_can_quant_stage(Ctx *c, int n_xrows, const W4Layout &L, int max_rows) {
    return max_rows <= 2 && gemv_rows_fit(c, n_xrows, L);
}

template <bool GROUPED, int BPG>
static int tile_launch_t(Ctx *c, const GemvParams &P) {
    auto kfn = ffn_w4a8_tile_kernel<GROUPED, BPG>;
    if (!ensure_smem(c, kfn, (size_t)kTileSmemBytes, "tile kernel shared-memory opt-in")) return 0;
    const int n_oblk = (P.mode == 0) ? (P.ntile + 3) / 4 : (P.ntile + 7) / 8;
    return launch(kfn, dim3(n_oblk, P.tile_rb), dim3(kTileThreads), (size_t)kTileSmemBytes, c->stream,
                  "w4a8 tile kernel launch", P);
}
template <bool GROUPED, int BPG>
static int umma_launch_t(Ctx *c, const GemvParams &P) {
    auto kfn = ffn_w4a8_umma_kernel<GROUPED, BPG>;
    if (!ensure_smem(c, kfn, (size_t)kUmSmemBytes, "tcgen05 kernel shared-memory opt-in")) return 0;
    const int n_oblk = (P.mode == 0) ? (P.ntile + 3) / 4 : (P.ntile + 7) / 8;
    return launch(kfn, dim3(n_oblk, P.tile_rb), dim3(kUmThreads), (size_t)kUmSmemBytes, c->stream,
                  "w4a8 tcgen05 kernel launch", P);
}
static int tile_launch(Ctx *c, const GemvParams &P, bool grouped, int bpg) {
    if (P.umma) {
        if (!grouped) return umma_launch_t<false, 1>(c, P);
        switch (bpg) {
            case 1: return umma_launch_t<true, 1>(c, P);
            case 2: return umma_launch_t<true, 2>(c, P);
            case 4: return umma_launch_t<true, 4>(c, P);
            case 8: return umma_launch_t<true, 8>(c, P);
        }
        return fail("w4a8 tcgen05 kernel: unsupported group size");
    }
    if (!grouped) return tile_launch_t<false, 1>(c, P);
    switch (bpg) {
        case 1: return tile_launch_t<true, 1>(c, P);
        case 2: return tile_launch_t<true, 2>(c, P);
        case 4: return tile_launch_t<true, 4>(c, P);
        case 8: return tile_launch_t<true, 8>(c, P);
    }
    return fail("w4a8 tile kernel: unsupported group size");
}

// Fills the layout-dependent fields and launches.  `max_rows` bounds the rows of any slot:
// up to 2 rows run the dp4a kernel, more run the tensor-core kernel.
// `want_quant_stage`: the caller filled x_f32 / amax_bits and wants the kernel to quantise the
// rows itself; only valid when gemv_can_quant_stage() said so.
static void gemv_fill_layout(Ctx *c, GemvParams &P, const W4Layout &L, int mode) {
    P.mode = mode;
    P.nchunk = L.nchunk;
    P.chunk_bytes = L.chunk_bytes;
    P.ntile = L.ntile;
    P.warp_tiles = (mode == 0) ? L.ntile : (L.ntile + 1) / 2;
    P.O = L.O;
    P.K = L.K;
    P.ng_tap = L.grouped ? L.ng_src : 1;
    P.tile_bytes = L.tile_bytes;
    P.xq_stride = L.kp;
    P.cs_stride = L.nblk;
    P.err = c->err_dev;
    P.neg_zero = -0.0f;
}

static int gemv_run(Ctx *c, GemvParams P, const W4Layout &L, int mode, int max_rows, bool want_quant_stage = false) {
    gemv_fill_layout(c, P, L, mode);
    const bool grouped = L.grouped != 0;
    if (P.tile_rb > 0) {
        if (want_quant_stage) return fail("w4a8 tile kernel: no quantising stage");
        if (P.pcap <= 0) return fail("w4a8 tile kernel: needs chunk-major activations");
        return tile_launch(c, P, grouped, L.bpg);
    }
    if (gemv_uses_mma(max_rows)) {
        if (want_quant_stage) return fail("w4a8 gemv: quantising stage is not available beyond 2 rows per expert");
        if (P.pcap <= 0) return fail("w4a8 gemv: the tensor-core kernel needs chunk-major activations");
        // experts with many rows: the warps of a CTA share the rows (no inspection taps on that path)
        if (!P.tap && P.comb.col_done == nullptr && max_rows >= block_min_rows()) return block_launch(c, P, grouped, L.bpg);
        if (max_rows <= 8) return mma_launch_r<1>(c, P, grouped, L.bpg);
        return mma_launch_r<2>(c, P, grouped, L.bpg);
    }
    const size_t base = (size_t)kRingBytes + kGemvBarBytes;
    const bool fit = gemv_rows_fit(c, P.n_xrows, L);
    const int xs = fit ? (want_quant_stage ? 2 : 1) : 0;
    if (want_quant_stage && !fit) return fail("w4a8 gemv: quantising stage requested but rows do not fit");
    const size_t smem = base + (fit ? gemv_xs_bytes(P.n_xrows, L.kp, L.nblk) : 0);
    if (max_rows <= 1) return gemv_launch_r<1>(c, P, grouped, L.bpg, xs, smem);
    return gemv_launch_r<2>(c, P, grouped, L.bpg, xs, smem);
}

// Loads and configures every kernel a single-matrix product (down-style launch, no taps, no
// quantising stage) of this weight format can reach, whatever the row count: the dp4a kernel for 1
// and 2 rows with and without staged activations, the tensor-core kernels for 8 and 16 rows per
// pass and for shared rows, the quantiser and the slot writer.  After this no later call on the device meets a first-use
// module load or a shared-memory opt-in for these kernels.
template <bool GROUPED, int BPG>
static int gemm_prepare_t(Ctx *c) {
    cudaFuncAttributes fa;
    int ok = 1;
    auto touch = [&](auto kfn, size_t smem, const char *what) {
        ok = ok && ensure_smem(c, kfn, smem, what) &&
             cuda_ok(cudaFuncGetAttributes(&fa, reinterpret_cast<const void *>(kfn)), what);
    };
    touch(gemv_w4a8_kernel<1, GROUPED, BPG, 0, false>, c->smem_optin, "gemv preparation");
    touch(gemv_w4a8_kernel<1, GROUPED, BPG, 1, false>, c->smem_optin, "gemv preparation");
    touch(gemv_w4a8_kernel<2, GROUPED, BPG, 0, false>, c->smem_optin, "gemv preparation");
    touch(gemv_w4a8_kernel<2, GROUPED, BPG, 1, false>, c->smem_optin, "gemv preparation");
    touch(gemv_w4a8_mma_kernel<1, GROUPED, BPG, false>, (size_t)mma_ring_bytes(1) + kMmaBarBytes, "mma gemv preparation");
    touch(gemv_w4a8_mma_kernel<2, GROUPED, BPG, false>, (size_t)mma_ring_bytes(2) + kMmaBarBytes, "mma gemv preparation");
    touch(gemv_w4a8_block_kernel<GROUPED, BPG>, (size_t)kBlkSmemBytes, "block gemv preparation");
    touch(qrow_i8_kernel, 0, "quantiser preparation");
    touch(write_slot_kernel, 0, "slot writer preparation");
    return ok;
}
static int gemm_prepare(Ctx *c, const W4Layout &L) {
    if (!L.grouped) return gemm_prepare_t<false, 1>(c);
    switch (L.bpg) {
        case 1: return gemm_prepare_t<true, 1>(c);
        case 2: return gemm_prepare_t<true, 2>(c);
        case 4: return gemm_prepare_t<true, 4>(c);
        case 8: return gemm_prepare_t<true, 8>(c);
    }
    return fail("w4a8 gemv: unsupported group size");
}

// The fused single-token decode step (kernels_decode.cuh): one CTA per SM.
template <bool GROUPED, int BPG>
static int decode_launch_t(Ctx *c, const DecodeArgs &A, size_t smem) {
    auto kfn = decode_step_kernel<GROUPED, BPG>;
    if (!ensure_smem(c, kfn, smem, "decode step shared-memory opt-in")) return 0;
    return launch(kfn, dim3(c->sms), dim3(kGemvThreads), smem, c->stream, "decode step launch", A);
}
static int decode_launch(Ctx *c, const DecodeArgs &A, const W4Layout &L, size_t smem) {
    if (!L.grouped) return decode_launch_t<false, 1>(c, A, smem);
    switch (L.bpg) {
        case 1: return decode_launch_t<true, 1>(c, A, smem);
        case 2: return decode_launch_t<true, 2>(c, A, smem);
        case 4: return decode_launch_t<true, 4>(c, A, smem);
        case 8: return decode_launch_t<true, 8>(c, A, smem);
    }
    return fail("decode step: unsupported group size");
}

// Quantises `grid_rows` (at most) fp32 rows.  pcap > 0 writes the chunk-major layout with that row
// capacity (tensor-core kernel), else the row-major layout (dp4a kernel).  rowmap (device, optional)
// names the source row of each output row.
static int qrow_run(Ctx *c, const float *x, long long ldx, int K, const W4Layout &L, int8_t *xq, float *sx, int *cs,
                    const int *n_rows_dev, int n_rows, int grid_rows, const int *rowmap = nullptr,
                    long long pcap = 0, const unsigned *amax_bits = nullptr) {
    if (grid_rows < 1) return 1;
    return launch(qrow_i8_kernel, dim3(grid_rows), dim3(256), 0, c->stream, "activation quantise launch", x, ldx, K,
                  L.kp, L.nblk, xq, sx, cs, n_rows_dev, n_rows, rowmap, pcap, amax_bits);
}

// ------------------------------------------------------------- expert group
// Shape cache counters of the reference's COLI_CUDA_GRAPH knob (cuda/backend_cuda.cu:678-745,
// 1110-1166).  The launch sequence of this backend is a handful of kernels whose arguments all
// come from device tables, so no graph is instantiated: a call takes the same path with the knob
// on or off and its result is bit-identical.  What the caller can observe through
// coli_cuda_graph_cache_stats is kept as the reference keeps it, as bookkeeping: the key is an
// FNV-1a hash of the launch shape (arm, count, D, I, the reduce / tile word, rows[]); the first
// call at a shape under the current scratch generation counts as a capture, a repeat as a
// replay; an entry recorded before any scratch buffer of the device grew is dropped on its next
// lookup and counted as an invalidation (the call then counts as a capture again); 16 entries per
// device, least recently used evicted; a call the reference would not cache (its W4A16 arm, or
// profiling on) counts as uncacheable.
static uint64_t shape_key(int arm, int count, int D, int I, const int *rows, long long extra) {
    uint64_t h = 1469598103934665603ULL;
    auto mix = [&h](uint64_t v) {
        for (int b = 0; b < 8; ++b) {
            h ^= (v >> (b * 8)) & 0xFF;
            h *= 1099511628211ULL;
        }
    };
    mix((uint64_t)arm);
    mix((uint64_t)count);
    mix((uint64_t)D);
    mix((uint64_t)I);
    mix((uint64_t)extra);
    for (int c = 0; c < count; ++c) mix((uint64_t)rows[c]);
    return h ? h : 1;  // 0 marks an empty entry
}
// Books one graph-knob call; the caller holds g_stats_mu.
static void shape_cache_note(Ctx *c, uint64_t key) {
    for (Ctx::ShapeSlot &e : c->shapes) {
        if (e.key != key) continue;
        if (e.gen == c->scratch_gen) {
            e.used = ++c->shape_clock;
            g_replays++;
            return;
        }
        e.key = 0;  // recorded against scratch that has since moved
        g_invalidations++;
        break;
    }
    Ctx::ShapeSlot *victim = &c->shapes[0];
    for (Ctx::ShapeSlot &e : c->shapes) {
        if (!e.key) {
            victim = &e;
            break;
        }
        if (e.used < victim->used) victim = &e;
    }
    victim->key = key;
    victim->gen = c->scratch_gen;
    victim->used = ++c->shape_clock;
    g_captures++;
}

struct ReduceSpec {
    const int *row_ptr, *row_idx;
    const float *rw;
    int s_n;
    float *out;
};

static bool same_class(const ColiCudaTensor *a, const ColiCudaTensor *b) {
    return a->kind == b->kind && a->gs == b->gs;
}

static int expert_group_impl(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                             const int *rows, int count, float *y, const float *x, const ReduceSpec *red,
                             int *arm_out, int tile_word = 0) {
    if (!gates || !ups || !downs || !rows || !x || count < 1 || count > 256) return 0;
    if (!red && !y) return 0;
    if (red && (!red->row_ptr || !red->row_idx || !red->rw || !red->out || red->s_n < 1)) return 0;
    ColiCudaTensor *first = gates[0];
    if (!first) return 0;
    const int device = first->device, D = first->I, I = first->O;
    int total = 0, max_rows = 0, all_i4 = 1, min_rows = 1 << 30;
    std::vector<int> row0(count);
    for (int cidx = 0; cidx < count; ++cidx) {
        ColiCudaTensor *g = gates[cidx], *u = ups[cidx], *d = downs[cidx];
        if (!g || !u || !d || rows[cidx] < 1 || g->device != device || u->device != device || d->device != device ||
            g->I != D || u->I != D || g->O != I || u->O != I || d->I != I || d->O != D)
            return 0;
        if (!same_class(g, u)) return fail("expert group: gate and up of one expert must share a format");
        all_i4 &= (g->kind != 0 && d->kind != 0);
        row0[cidx] = total;
        total += rows[cidx];
        max_rows = rows[cidx] > max_rows ? rows[cidx] : max_rows;
        min_rows = rows[cidx] < min_rows ? rows[cidx] : min_rows;
    }
    Ctx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    // The arm code the reference's selector would report for this call
    // (cuda/backend_cuda.cu:897-930): 1 when the W4A16 knob is on and the group
    // qualifies, 2 for all-int4 groups, 3 otherwise.  One kernel family serves all.
    int arm = all_i4 ? 2 : 3;
    if (all_i4 && env_flag("COLI_CUDA_TC_W4A16", 0) && min_rows >= env_flag("COLI_CUDA_TC_W4A16_MIN", 16)) arm = 1;
    if (arm_out) *arm_out = arm;

    const size_t xb = (size_t)total * D * 4, hb = (size_t)total * I * 4;
    W4Layout Lx, Lh;  // activation layouts (per-row kind: padding to 32 only)
    w4_layout_make(&Lx, 1, D, 0, 0);
    w4_layout_make(&Lh, 1, I, 0, 0);
    // grouped formats may pad K up to a multiple of gs: size for the largest gs (256)
    const size_t kpx = ((size_t)D + 255) / 256 * 256 + 256, kph = ((size_t)I + 255) / 256 * 256 + 256;
    if (!reserve(c, c->x, xb) || !reserve(c, c->y, xb) || !reserve(c, c->h, hb) ||
        !reserve(c, c->xq, (size_t)total * kpx * 17 / 16 + 512) || !reserve(c, c->sx, (size_t)total * 4) ||
        !reserve(c, c->xcs, (size_t)total * (kpx / 32) * 4) || !reserve(c, c->hq, (size_t)total * kph * 17 / 16 + 512) ||
        !reserve(c, c->sh, (size_t)total * 4) || !reserve(c, c->hcs, (size_t)total * (kph / 32) * 4) ||
        !reserve(c, c->pin_x, xb, true) || !reserve(c, c->pin_y, xb, true))
        return 0;
    const int profile = env_flag("COLI_CUDA_PROFILE", 0);
    const int graph_knob = env_flag("COLI_CUDA_GRAPH", 0);
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    if (profile)
        for (auto &e : ev) cudaEventCreate(&e);
    int ok = 1;
    std::memcpy(c->pin_x.p, x, xb);
    if (profile) cudaEventRecord(ev[0], c->stream);
    ok = ok && cuda_ok(cudaMemcpyAsync(c->x.p, c->pin_x.p, xb, cudaMemcpyHostToDevice, c->stream), "group x upload");
    if (profile) cudaEventRecord(ev[1], c->stream);

    // ---- slot tables of every format class of both phases, built up front in one page-locked
    // block (count at +0, table at +16 of each class's region) and uploaded with a single
    // asynchronous copy ahead of the first launch: nothing in this call waits for the stream
    // before the final synchronise.
    struct ClassLaunch {
        int phase;  // 0: gate/up, 1: down
        const ColiCudaTensor *cls;
        int cls_max, n;
        size_t off;  // byte offset of the region inside the block
    };
    std::vector<ClassLaunch> classes;
    std::vector<unsigned char> blob;
    for (int phase = 0; phase < 2; ++phase) {
        ColiCudaTensor *const *lead_of = phase == 0 ? gates : downs;
        std::vector<char> done(count, 0);
        for (int lead = 0; lead < count; ++lead) {
            if (done[lead]) continue;
            const ColiCudaTensor *cls = lead_of[lead];
            ClassLaunch cl{phase, cls, 0, 0, (blob.size() + 255) & ~(size_t)255};
            blob.resize(cl.off + 16);
            for (int j = lead; j < count; ++j) {
                if (done[j] || !same_class(lead_of[j], cls)) continue;
                done[j] = 1;
                cl.cls_max = rows[j] > cl.cls_max ? rows[j] : cl.cls_max;
                cl.n++;
                const size_t at = blob.size();
                if (cls->kind == 0) {
                    const F32Slot f = phase == 0 ? F32Slot{(const float *)gates[j]->data, (const float *)ups[j]->data,
                                                           row0[j], rows[j]}
                                                 : F32Slot{(const float *)downs[j]->data, nullptr, row0[j], rows[j]};
                    blob.resize(at + sizeof(F32Slot));
                    std::memcpy(blob.data() + at, &f, sizeof(F32Slot));
                } else {
                    const GemvSlot g = phase == 0
                                           ? GemvSlot{(const uint8_t *)gates[j]->data, (const uint8_t *)ups[j]->data,
                                                      gates[j]->row_scales, ups[j]->row_scales, row0[j], rows[j]}
                                           : GemvSlot{(const uint8_t *)downs[j]->data, nullptr, downs[j]->row_scales,
                                                      nullptr, row0[j], rows[j]};
                    blob.resize(at + sizeof(GemvSlot));
                    std::memcpy(blob.data() + at, &g, sizeof(GemvSlot));
                }
            }
            std::memcpy(blob.data() + cl.off, &cl.n, sizeof(int));
            classes.push_back(cl);
        }
    }
    ok = ok && reserve(c, c->slots_gu, blob.size()) && reserve(c, c->pin_slots, blob.size(), true);
    if (ok) {
        std::memcpy(c->pin_slots.p, blob.data(), blob.size());
        ok = cuda_ok(cudaMemcpyAsync(c->slots_gu.p, c->pin_slots.p, blob.size(), cudaMemcpyHostToDevice, c->stream),
                     "group slot upload");
    }
    // ---- phase 1: gate/up (+ SwiGLU) into h; phase 2: down into y; one launch per format class
    for (size_t ci = 0; ok && ci < classes.size(); ++ci) {
        const ClassLaunch &cl = classes[ci];
        const unsigned char *region = (const unsigned char *)c->slots_gu.p + cl.off;
        const bool up = cl.phase == 0;
        if (cl.cls->kind == 0) {
            ok = up ? launch(gemv_f32_kernel, dim3((I + 7) / 8, cl.cls_max, cl.n), dim3(256), 0, c->stream,
                             "f32 gate/up launch", (const F32Slot *)(region + 16), cl.n, 0, I, D,
                             (const float *)c->x.p, (long long)D, (float *)c->h.p, (long long)I, cl.cls_max)
                    : launch(gemv_f32_kernel, dim3((D + 7) / 8, cl.cls_max, cl.n), dim3(256), 0, c->stream,
                             "f32 down launch", (const F32Slot *)(region + 16), cl.n, 1, D, I, (const float *)c->h.p,
                             (long long)I, (float *)c->y.p, (long long)D, cl.cls_max);
            continue;
        }
        const W4Layout &L = cl.cls->L;
        ok = up ? qrow_run(c, (const float *)c->x.p, D, D, L, (int8_t *)c->xq.p, (float *)c->sx.p, (int *)c->xcs.p,
                           nullptr, total, total, nullptr, gemv_uses_mma(cl.cls_max) ? total : 0)
                : qrow_run(c, (const float *)c->h.p, I, I, L, (int8_t *)c->hq.p, (float *)c->sh.p, (int *)c->hcs.p,
                           nullptr, total, total, nullptr, gemv_uses_mma(cl.cls_max) ? total : 0);
        GemvParams P{};
        P.slots = (const GemvSlot *)(region + 16);
        P.n_slots = (const int *)region;
        P.xq = (const int8_t *)(up ? c->xq.p : c->hq.p);
        P.csum = (const int *)(up ? c->xcs.p : c->hcs.p);
        P.sx = (const float *)(up ? c->sx.p : c->sh.p);
        P.rowmap = nullptr;
        P.n_xrows = total;
        P.pcap = total;
        P.out = (float *)(up ? c->h.p : c->y.p);
        P.out_stride = up ? I : D;
        ok = ok && gemv_run(c, P, L, up ? 0 : 1, cl.cls_max);
    }
    // ---- optional CSR combine, then the result back to the host
    size_t out_bytes = xb;
    const void *out_dev = c->y.p;
    if (ok && red) {
        out_bytes = (size_t)red->s_n * D * 4;
        ok = reserve(c, c->csr_ptr, (size_t)(red->s_n + 1) * 4) && reserve(c, c->csr_idx, (size_t)total * 4) &&
             reserve(c, c->csr_rw, (size_t)total * 4) && reserve(c, c->out, out_bytes) &&
             reserve(c, c->pin_y, out_bytes > xb ? out_bytes : xb, true) &&
             cuda_ok(cudaMemcpyAsync(c->csr_ptr.p, red->row_ptr, (size_t)(red->s_n + 1) * 4, cudaMemcpyHostToDevice,
                                     c->stream),
                     "reduce layout upload") &&
             cuda_ok(cudaMemcpyAsync(c->csr_idx.p, red->row_idx, (size_t)total * 4, cudaMemcpyHostToDevice, c->stream),
                     "reduce layout upload") &&
             cuda_ok(cudaMemcpyAsync(c->csr_rw.p, red->rw, (size_t)total * 4, cudaMemcpyHostToDevice, c->stream),
                     "reduce weights upload") &&
             launch(csr_reduce_kernel, dim3((D + 255) / 256, red->s_n), dim3(256), 0, c->stream, "csr reduce launch",
                    (const float *)c->y.p, D, (const int *)c->csr_ptr.p, (const int *)c->csr_idx.p,
                    (const float *)c->csr_rw.p, (float *)c->out.p);
        out_dev = c->out.p;
    }
    if (profile) cudaEventRecord(ev[2], c->stream);
    ok = ok && cuda_ok(cudaMemcpyAsync(c->pin_y.p, out_dev, out_bytes, cudaMemcpyDeviceToHost, c->stream),
                       "group result download");
    if (profile) cudaEventRecord(ev[3], c->stream);
    ok = cuda_ok(cudaStreamSynchronize(c->stream), "group synchronize") && ok;
    if (ok) std::memcpy(red ? (void *)red->out : (void *)y, c->pin_y.p, out_bytes);
    if (ok) {
        const int dev_err = *static_cast<volatile int *>(c->err_dev);
        if (dev_err) {
            *static_cast<volatile int *>(c->err_dev) = 0;
            std::fprintf(stderr, "[CUDA] expert group: device reported error %d\n", dev_err);
            ok = 0;
        }
    }
    {
        std::lock_guard<std::mutex> lk(g_stats_mu);
        g_calls++;
        g_experts += (uint64_t)count;
        g_rows += (uint64_t)total;
        if (profile && ok) {
            float a = 0, b = 0, d = 0;
            cudaEventElapsedTime(&a, ev[0], ev[1]);
            cudaEventElapsedTime(&b, ev[1], ev[2]);
            cudaEventElapsedTime(&d, ev[2], ev[3]);
            g_h2d_ms += a;
            g_kernel_ms += b;
            g_d2h_ms += d;
        }
        if (graph_knob) {
            if (arm != 1 && !profile && ok)
                shape_cache_note(c, shape_key(arm, count, D, I, rows,
                                              (long long)(red ? red->s_n : -1) * 1000003 + tile_word));
            else
                g_uncacheable++;
        }
    }
    if (profile)
        for (auto &e : ev) cudaEventDestroy(e);
    return ok;
}

PGB_EXPORT int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                      ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                                      const float *x) {
    return expert_group_impl(gates, ups, downs, rows, count, y, x, nullptr, nullptr);
}
PGB_EXPORT int coli_cuda_expert_group_tiled(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                            ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                                            const float *x, int tile_m, int tile_n, int tile_k, int *arm_out) {
    // the tile only separates shape-cache entries here (one kernel family serves every tile)
    return expert_group_impl(gates, ups, downs, rows, count, y, x, nullptr, arm_out,
                             tile_m * 10007 + tile_n * 101 + tile_k);
}
PGB_EXPORT int coli_cuda_expert_group_reduce(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                             ColiCudaTensor *const *downs, const int *rows, int count,
                                             const int *row_ptr, const int *row_idx, const float *rw, int s_n,
                                             float *out, const float *x) {
    ReduceSpec red = {row_ptr, row_idx, rw, s_n, out};
    return expert_group_impl(gates, ups, downs, rows, count, nullptr, x, &red, nullptr);
}

PGB_EXPORT int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                    const float *x, int S) {
    if (S < 1) return 0;
    return expert_group_impl(&gate, &up, &down, &S, 1, y, x, nullptr, nullptr);
}
PGB_EXPORT int coli_cuda_shared_mlp_w4a16(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                          const float *x, int S) {
    return coli_cuda_expert_mlp(gate, up, down, y, x, S);
}

namespace pgb {
__global__ void pipe_add_kernel(float *x, const float *t, size_t n);  // defined with the other pipe kernels
}

#include "backend_layer.inc"
#include "backend_pipe.inc"
#include "backend_noalloc.inc"
#include "backend_ep.inc"
