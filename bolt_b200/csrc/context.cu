// context.cu -- per-device state, the staging of host pointers, and the runtime entry points.
#include <cstring>

#include "common.cuh"

namespace b200 {

std::atomic<uint64_t> g_launches{0};

namespace {
constexpr int kMaxDevices = 16;
DeviceCtx *g_ctx[kMaxDevices] = {nullptr};
std::mutex g_ctx_mu;
constexpr size_t kWorkspaceMin = 64ull << 20;
}  // namespace

ThreadState &tls()
{
    static thread_local ThreadState s;
    return s;
}

EE cuda_ee(cudaError_t e)
{
    switch (e) {
        case cudaSuccess:
            return SUCCESS;
        case cudaErrorMemoryAllocation:
            return ALLOC_FAILED;
        case cudaErrorInvalidValue:
            return NOT_MATCH;
        default:
            return UNKNOWN;
    }
}

DeviceCtx *ctx()
{
    // The device chosen with bolt_b200_set_device, else the CUDA device that is current in this thread (a
    // caller that manages devices itself -- one rank per GPU under torch.distributed -- is followed, not
    // overridden).
    int dev = tls().device;
    if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        return nullptr;
    }
    {
        // fast path: the context exists and its device is current
        DeviceCtx *c = __atomic_load_n(&g_ctx[dev], __ATOMIC_ACQUIRE);
        if (c != nullptr) {
            int cur = -1;
            if (cudaGetDevice(&cur) != cudaSuccess || cur != dev) {
                cudaSetDevice(dev);
            }
            return c;
        }
    }
    std::lock_guard<std::mutex> g(g_ctx_mu);
    if (g_ctx[dev] == nullptr) {
        if (cudaSetDevice(dev) != cudaSuccess) {
            return nullptr;
        }
        DeviceCtx *c = new DeviceCtx();
        c->device = dev;
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
            c->sm_count = prop.multiProcessorCount;
        }
        if (cudaMalloc(&c->d_status, 256) != cudaSuccess ||
            cudaMemset(c->d_status, 0, 256) != cudaSuccess ||
            cudaMalloc(&c->d_scratch, 4096) != cudaSuccess) {
            delete c;
            return nullptr;
        }
        c->d_scratch_u = reinterpret_cast<unsigned *>(c->d_scratch);
        cudaMemset(c->d_scratch, 0, 4096);
        __atomic_store_n(&g_ctx[dev], c, __ATOMIC_RELEASE);
    } else {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != dev) {
            cudaSetDevice(dev);
        }
    }
    return g_ctx[dev];
}

EE raise_smem_limit(DeviceCtx *c, KernelFamily f, const void *const *kernels, int n, size_t bytes)
{
    std::lock_guard<std::mutex> g(c->attr_mu);
    if (c->smem_raised[f]) {
        return SUCCESS;
    }
    for (int i = 0; i < n; ++i) {
        B200_CUDA(cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    c->smem_raised[f] = true;
    return SUCCESS;
}

bool is_device_ptr(const void *p)
{
    if (p == nullptr) {
        return false;
    }
    if (tls().device_only) {
        return true;
    }
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

bool on_other_device(const void *p)
{
    if (p == nullptr || tls().device_only) {
        return false;
    }
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (a.type != cudaMemoryTypeDevice) {
        return false;
    }
    int dev = tls().device;
    if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.device != dev;
}

// ---- Stage -----------------------------------------------------------------------------------
Stage::Stage() {}

Stage::~Stage()
{
    for (void *p : big_) {
        cudaFree(p);
    }
    if (locked_) {
        DeviceCtx *c = ctx();
        c->ws_used = 0;
        c->mu.unlock();
    }
}

void *Stage::alloc(size_t bytes)
{
    DeviceCtx *c = ctx();
    if (!locked_) {
        c->mu.lock();  // the workspace belongs to one staged call at a time
        locked_ = true;
        c->ws_used = 0;
    }
    bytes = B200_ALIGN(bytes, 256);
    if (c->ws == nullptr) {
        if (cudaMalloc(&c->ws, kWorkspaceMin) == cudaSuccess) {
            c->ws_bytes = kWorkspaceMin;
        } else {
            cudaGetLastError();
            c->ws = nullptr;
        }
    }
    if (c->ws != nullptr && c->ws_used + bytes <= c->ws_bytes) {
        void *p = c->ws + c->ws_used;
        c->ws_used += bytes;
        return p;
    }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    big_.push_back(p);
    return p;
}

const void *Stage::in(const void *p, size_t bytes)
{
    if (p == nullptr || bytes == 0 || is_device_ptr(p)) {
        return p;
    }
    any_host_ = true;
    void *d = alloc(bytes);
    if (d == nullptr) {
        return nullptr;
    }
    if (cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, tls().stream) != cudaSuccess) {
        return nullptr;
    }
    return d;
}

void *Stage::out(void *p, size_t bytes, bool also_in)
{
    if (p == nullptr || bytes == 0 || is_device_ptr(p)) {
        return p;
    }
    any_host_ = true;
    void *d = alloc(bytes);
    if (d == nullptr) {
        return nullptr;
    }
    if (also_in &&
        cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, tls().stream) != cudaSuccess) {
        return nullptr;
    }
    outs_.push_back({p, d, bytes});
    return d;
}

void *Stage::scratch(size_t bytes)
{
    return alloc(bytes);
}

EE Stage::finish()
{
    cudaStream_t st = tls().stream;
    for (const Out &o : outs_) {
        B200_CUDA(cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, st));
    }
    if (any_host_ || !big_.empty() || locked_) {
        B200_CUDA(cudaStreamSynchronize(st));
    }
    return SUCCESS;
}

}  // namespace b200

using namespace b200;

extern "C" {

EE bolt_b200_set_device(int device)
{
    int n = 0;
    B200_CUDA(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n || device >= kMaxDevices) {
        return NOT_FOUND;
    }
    tls().device = device;
    return ctx() ? SUCCESS : UNKNOWN;
}

EE bolt_b200_use_para(const bolt_b200_para *para)
{
    if (para == nullptr) {
        tls().device = -1;
        tls().stream = nullptr;
        return SUCCESS;
    }
    B200_EE(bolt_b200_set_device(para->device));
    tls().stream = reinterpret_cast<cudaStream_t>(para->stream);
    return SUCCESS;
}

// ---- buffers shared between the processes of one box (one process per GPU) ----------------------------
// export: a handle for a buffer obtained from bolt_b200_malloc; import: the peer's buffer as a pointer this
// process may store to (peer access is enabled by the import); close: unmap it.
EE bolt_b200_ipc_export(void *p, void *handle64)
{
    if (p == nullptr || handle64 == nullptr) {
        return NULL_POINTER;
    }
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    B200_CUDA(cudaIpcGetMemHandle(&h, p));
    std::memcpy(handle64, &h, sizeof(h));
    return SUCCESS;
}

EE bolt_b200_ipc_import(const void *handle64, void **p)
{
    if (p == nullptr || handle64 == nullptr) {
        return NULL_POINTER;
    }
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    B200_CUDA(cudaIpcOpenMemHandle(p, h, cudaIpcMemLazyEnablePeerAccess));
    return SUCCESS;
}

EE bolt_b200_ipc_close(void *p)
{
    if (p == nullptr) {
        return NULL_POINTER;
    }
    B200_CUDA(cudaIpcCloseMemHandle(p));
    return SUCCESS;
}

EE bolt_b200_set_stream(void *cuda_stream)
{
    tls().stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    return SUCCESS;
}

int bolt_b200_device_status(void)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return -1;
    }
    int v = 0;
    if (cudaMemcpy(&v, c->d_status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        return -1;
    }
    if (v != 0) {
        cudaMemset(c->d_status, 0, sizeof(int));
    }
    return v;
}

EE bolt_b200_synchronize(void)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    B200_CUDA(cudaStreamSynchronize(tls().stream));
    return bolt_b200_device_status() == 0 ? SUCCESS : UNKNOWN;
}

EE bolt_b200_set_pointer_mode(int device_only)
{
    tls().device_only = (device_only != 0);
    return SUCCESS;
}

void *bolt_b200_malloc(size_t bytes)
{
    if (ctx() == nullptr) {
        return nullptr;
    }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void bolt_b200_free(void *p)
{
    if (p != nullptr) {
        cudaFree(p);
    }
}

EE bolt_b200_memcpy_h2d(void *dst, const void *src, size_t bytes)
{
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, tls().stream));
    B200_CUDA(cudaStreamSynchronize(tls().stream));
    return SUCCESS;
}

EE bolt_b200_memcpy_d2h(void *dst, const void *src, size_t bytes)
{
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, tls().stream));
    B200_CUDA(cudaStreamSynchronize(tls().stream));
    return SUCCESS;
}

EE bolt_b200_release_weight(const void *host_packed)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    std::lock_guard<std::mutex> g(c->twin_mu);
    auto it = c->twins.find(host_packed);
    if (it == c->twins.end()) {
        return NOT_FOUND;
    }
    cudaFree(it->second.dev);
    c->twins.erase(it);
    return SUCCESS;
}

uint64_t bolt_b200_launch_count(void)
{
    return g_launches.load();
}

int bolt_b200_last_gemm_used_tensor_cores(void)
{
    return tls().last_gemm_tc;
}

}  // extern "C"
