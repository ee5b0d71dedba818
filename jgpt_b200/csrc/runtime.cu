// Context, stream, device buffers, events, error reporting.
#include "common.cuh"

#include <cmath>
#include <cstdlib>

#include <cstdlib>

namespace jgpt {

std::string &last_error_ref() {
    static thread_local std::string s;
    return s;
}

int32_t fail(int32_t code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

Registry<Ctx> &ctx_registry() {
    static Registry<Ctx> r;
    return r;
}
Registry<Pool> &pool_registry() {
    static Registry<Pool> r;
    return r;
}

cudaError_t status_enqueue_read(Ctx *c) {
    return cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream);
}

// To be called after the stream has been synchronised behind status_enqueue_read.  A non-zero word means a kernel of
// the step recorded a self-check failure (its results are not to be trusted): the word is cleared, the pool's split-K
// arrival counters and work-queue counters are put back to zero (an aborted launch can leave them half counted, which
// would make every later launch on the pool merge too early or never), and the call fails.
int32_t status_check_after_sync(Ctx *c, Pool *p, const char *what) {
    const int st = *c->h_status;
    if (st == 0) return JGPT_OK;
    *c->h_status = 0;
    cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream);
    if (p) {
        if (p->d_tickets && p->n_tickets) cudaMemsetAsync(p->d_tickets, 0, sizeof(int) * p->n_tickets, c->stream);
        if (p->d_item_counters) cudaMemsetAsync(p->d_item_counters, 0, sizeof(int) * 2, c->stream);
    }
    return fail(JGPT_ERR_DEVICE_CHECK, "%s: device self-check failed: status=0x%x%s%s%s%s%s", what, st,
                (st & DEV_STATUS_BAD_BLOCK) ? " bad-block-id" : "", (st & DEV_STATUS_BAD_POSITION) ? " bad-position" : "",
                (st & DEV_STATUS_BAD_SEQ) ? " bad-seq-id" : "", (st & DEV_STATUS_WAIT_TIMEOUT) ? " wait-timeout" : "",
                (st & DEV_STATUS_LEN_OVER_BOUND) ? " len-over-bound" : "");
}

int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    if (!v || !*v) return dflt;
    char *end = nullptr;
    long x = strtol(v, &end, 10);
    return (end && *end == 0) ? (int)x : dflt;
}

}  // namespace jgpt

using namespace jgpt;

extern "C" {

const char *jgpt_last_error(void) { return last_error_ref().c_str(); }

int32_t jgpt_device_count(int32_t *out) {
    JGPT_REQUIRE(out, JGPT_ERR_INVALID_ARGUMENT, "out is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *out = n;
    return JGPT_OK;
}

int32_t jgpt_ctx_create(int32_t device, jgpt_ctx *out) {
    JGPT_REQUIRE(out, JGPT_ERR_INVALID_ARGUMENT, "out is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        // The reference throws IllegalStateException from requireCuda when no GPU is usable.
        return fail(JGPT_ERR_ILLEGAL_STATE, "no CUDA device available (%s); this library has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
    }
    JGPT_REQUIRE(device >= 0 && device < n, JGPT_ERR_INVALID_ARGUMENT, "device %d outside [0,%d)", device, n);
    JGPT_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    JGPT_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    JGPT_REQUIRE(prop.major >= 10, JGPT_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                 device, prop.major, prop.minor);
    Ctx *c = new Ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    JGPT_CUDA_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    JGPT_CUDA_TRY(cudaMalloc(&c->d_status, sizeof(int)));
    JGPT_CUDA_TRY(cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream));
    JGPT_CUDA_TRY(cudaHostAlloc(&c->h_status, sizeof(int), cudaHostAllocDefault));
    *c->h_status = 0;
    JGPT_CUDA_TRY(cudaStreamSynchronize(c->stream));
    *out = ctx_registry().add(c);
    return JGPT_OK;
}

int32_t jgpt_ctx_destroy(jgpt_ctx h) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    make_current(c);
    cudaStreamSynchronize(c->stream);
    ctx_registry().remove(c);
    cudaFree(c->d_status);
    cudaFreeHost(c->h_status);
    cudaStreamDestroy(c->stream);
    delete c;
    return JGPT_OK;
}

int32_t jgpt_sync(jgpt_ctx h) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(status_enqueue_read(c));
    JGPT_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return status_check_after_sync(c, nullptr, "jgpt_sync");
}

// TensorOpsGPU.getGpuMemoryAllocated0 / getGpuMemoryReserved0 (src/main/cpp/jgpt_cuda_jni_ops_graph.inl:471-491):
// both are cudaMemGetInfo of the current device.
int32_t jgpt_mem_info(jgpt_ctx h, uint64_t *free_bytes_out, uint64_t *total_bytes_out) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_CUDA_TRY(make_current(c));
    size_t f = 0, t = 0;
    JGPT_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_bytes_out) *free_bytes_out = f;
    if (total_bytes_out) *total_bytes_out = t;
    return JGPT_OK;
}

// The JGPT_* settings that reach this path, read the way the reference reads them (env first, unparsable or
// out-of-range values ignored): JGPT_RMSNORM_EPS accepts 0 < v <= 1e-2 and otherwise falls back to 1e-5 with
// JGPT_FP16_MATMUL on, 1e-6 without (src/main/java/com/veles/llm/jgpt/TensorOpsGpuInit.java:30-101);
// JGPT_MAX_SEQ_LEN is a positive override of the configured context (training/LLMConfig.java:190-199).
// JGPT_KV_BLOCK_TOKENS (default 16), JGPT_KV_POOL_BLOCKS (0 = one full context per sequence) and
// JGPT_KV_BACKEND ("b200", the default, or anything else to keep the reference's own KV path) belong to this library.
int32_t jgpt_env_config(int32_t *kv_block_tokens_out, int32_t *kv_pool_blocks_out, int32_t *max_seq_len_out, float *rmsnorm_eps_out,
                        int32_t *backend_b200_out) {
    auto trimmed = [](const char *name) -> std::string {
        const char *v = getenv(name);
        if (!v) return std::string();
        std::string t(v);
        const size_t a = t.find_first_not_of(" \t\r\n"), b = t.find_last_not_of(" \t\r\n");
        return a == std::string::npos ? std::string() : t.substr(a, b - a + 1);
    };
    auto positive_int = [&](const char *name, int dflt) {
        const std::string t = trimmed(name);
        if (t.empty()) return dflt;
        char *end = nullptr;
        const long v = strtol(t.c_str(), &end, 10);
        return (end && *end == 0 && v > 0 && v <= 0x7fffffffL) ? (int)v : dflt;
    };
    auto truthy = [&](const char *name) {
        std::string t = trimmed(name);
        for (auto &ch : t) ch = (char)tolower((unsigned char)ch);
        return t == "1" || t == "true";
    };
    if (kv_block_tokens_out) *kv_block_tokens_out = positive_int("JGPT_KV_BLOCK_TOKENS", kBlockTokens);
    if (kv_pool_blocks_out) *kv_pool_blocks_out = positive_int("JGPT_KV_POOL_BLOCKS", 0);
    if (max_seq_len_out) *max_seq_len_out = positive_int("JGPT_MAX_SEQ_LEN", 0);
    if (rmsnorm_eps_out) {
        float eps = truthy("JGPT_FP16_MATMUL") ? 1e-5f : 1e-6f;
        const std::string t = trimmed("JGPT_RMSNORM_EPS");
        if (!t.empty()) {
            char *end = nullptr;
            const float v = strtof(t.c_str(), &end);
            if (end && *end == 0 && v > 0.f && std::isfinite(v) && v <= 1e-2f) eps = v;
        }
        *rmsnorm_eps_out = eps;
    }
    if (backend_b200_out) {
        std::string t = trimmed("JGPT_KV_BACKEND");
        for (auto &ch : t) ch = (char)tolower((unsigned char)ch);
        *backend_b200_out = (t.empty() || t == "b200") ? 1 : 0;
    }
    return JGPT_OK;
}

// PCI address of a device ("0000:1b:00.0"): lets a host pin its thread and its page-locked buffers to the NUMA
// node the GPU hangs off (/sys/bus/pci/devices/<id>/numa_node) before it allocates them.
int32_t jgpt_device_pci_bus_id(int32_t device, char *out, int32_t cap) {
    JGPT_REQUIRE(out && cap >= 16, JGPT_ERR_INVALID_ARGUMENT, "the bus id needs a buffer of at least 16 bytes");
    const cudaError_t e = cudaDeviceGetPCIBusId(out, cap, device);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(JGPT_ERR_INVALID_ARGUMENT, "device %d: %s", device, cudaGetErrorString(e));
    }
    for (char *c = out; *c; c++) *c = (char)tolower((unsigned char)*c);
    return JGPT_OK;
}

int32_t jgpt_ctx_stream(jgpt_ctx h, void **stream_out) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(stream_out, JGPT_ERR_INVALID_ARGUMENT, "stream_out is null");
    *stream_out = (void *)c->stream;
    return JGPT_OK;
}

int32_t jgpt_dev_alloc(jgpt_ctx h, uint64_t bytes, void **dev_out) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(dev_out && bytes > 0, JGPT_ERR_INVALID_ARGUMENT, "bytes must be > 0");
    JGPT_CUDA_TRY(make_current(c));
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(JGPT_ERR_OUT_OF_MEMORY, "cudaMalloc(%llu) failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    }
    *dev_out = p;
    return JGPT_OK;
}

int32_t jgpt_dev_free(jgpt_ctx h, void *dev) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    if (!dev) return JGPT_OK;
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaStreamSynchronize(c->stream));
    JGPT_CUDA_TRY(cudaFree(dev));
    return JGPT_OK;
}

int32_t jgpt_h2d(jgpt_ctx h, void *dev_dst, const void *host_src, uint64_t bytes) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    if (bytes == 0) return JGPT_OK;
    JGPT_REQUIRE(dev_dst && host_src, JGPT_ERR_INVALID_ARGUMENT, "null pointer");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, c->stream));
    // Pageable sources are staged by the runtime before the call returns; pinned ones are not,
    // so the caller's buffer must stay untouched until the stream passes this point.
    return JGPT_OK;
}

int32_t jgpt_d2h(jgpt_ctx h, void *host_dst, const void *dev_src, uint64_t bytes) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    if (bytes == 0) return JGPT_OK;
    JGPT_REQUIRE(host_dst && dev_src, JGPT_ERR_INVALID_ARGUMENT, "null pointer");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, c->stream));
    JGPT_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return JGPT_OK;
}

int32_t jgpt_dev_memset(jgpt_ctx h, void *dev, int32_t byte_value, uint64_t bytes) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    if (bytes == 0) return JGPT_OK;
    JGPT_REQUIRE(dev, JGPT_ERR_INVALID_ARGUMENT, "null pointer");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaMemsetAsync(dev, byte_value, bytes, c->stream));
    return JGPT_OK;
}

int32_t jgpt_host_alloc_pinned(uint64_t bytes, void **host_out) {
    JGPT_REQUIRE(host_out && bytes > 0, JGPT_ERR_INVALID_ARGUMENT, "bytes must be > 0");
    void *p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, bytes, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(JGPT_ERR_OUT_OF_MEMORY, "cudaHostAlloc(%llu) failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    }
    *host_out = p;
    return JGPT_OK;
}

int32_t jgpt_host_free_pinned(void *host) {
    if (!host) return JGPT_OK;
    JGPT_CUDA_TRY(cudaFreeHost(host));
    return JGPT_OK;
}

int32_t jgpt_event_create(uint64_t *event_out) {
    JGPT_REQUIRE(event_out, JGPT_ERR_INVALID_ARGUMENT, "event_out is null");
    cudaEvent_t e;
    JGPT_CUDA_TRY(cudaEventCreate(&e));
    *event_out = reinterpret_cast<uint64_t>(e);
    return JGPT_OK;
}

int32_t jgpt_event_destroy(uint64_t event) {
    if (!event) return JGPT_OK;
    JGPT_CUDA_TRY(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
    return JGPT_OK;
}

int32_t jgpt_event_record(jgpt_ctx h, uint64_t event) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(event, JGPT_ERR_INVALID_ARGUMENT, "null event");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), c->stream));
    return JGPT_OK;
}

int32_t jgpt_event_elapsed_ms(uint64_t start, uint64_t stop, float *ms_out) {
    JGPT_REQUIRE(start && stop && ms_out, JGPT_ERR_INVALID_ARGUMENT, "null argument");
    JGPT_CUDA_TRY(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(stop)));
    JGPT_CUDA_TRY(cudaEventElapsedTime(ms_out, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(stop)));
    return JGPT_OK;
}

// ---- CUDA graphs (TensorOpsGPU.cudaStreamBeginCapture0 / cudaStreamEndCaptureAndInstantiate0 /
// cudaGraphExecLaunch0 / cudaGraphExecDestroy0, src/main/cpp/jgpt_cuda_jni_ops_graph.inl:185-460) ----
int32_t jgpt_graph_begin_capture(jgpt_ctx h) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    return JGPT_OK;
}

int32_t jgpt_graph_end_capture(jgpt_ctx h, uint64_t *graph_exec_out) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(graph_exec_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    JGPT_CUDA_TRY(make_current(c));
    cudaGraph_t g = nullptr;
    JGPT_CUDA_TRY(cudaStreamEndCapture(c->stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(JGPT_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    *graph_exec_out = reinterpret_cast<uint64_t>(ex);
    return JGPT_OK;
}

int32_t jgpt_graph_launch(jgpt_ctx h, uint64_t graph_exec) {
    Ctx *c = ctx_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(graph_exec, JGPT_ERR_INVALID_ARGUMENT, "null graph");
    JGPT_CUDA_TRY(make_current(c));
    JGPT_CUDA_TRY(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_exec), c->stream));
    return JGPT_OK;
}

int32_t jgpt_graph_destroy(uint64_t graph_exec) {
    if (!graph_exec) return JGPT_OK;
    JGPT_CUDA_TRY(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph_exec)));
    return JGPT_OK;
}

}  // extern "C"
