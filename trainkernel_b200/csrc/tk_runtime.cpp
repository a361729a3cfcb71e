// libtrainkernel_rt.so: C ABI over the CUDA driver API (see include/trainkernel_rt.h).
//
// The driver library is opened with dlopen on first use, so this file links
// against nothing but libdl and can be loaded on a machine without a GPU.
#include "trainkernel_rt.h"

#include <cuda.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
    return code;
}

#define TK_STR2(x) #x
#define TK_STR(x) TK_STR2(x)
#define TK_DRIVER_SYMBOLS(X)                                                                        \
    X(cuInit) X(cuDeviceGet) X(cuDeviceGetAttribute) X(cuDevicePrimaryCtxRetain)                    \
    X(cuDevicePrimaryCtxRelease) X(cuCtxPushCurrent) X(cuCtxPopCurrent) X(cuCtxSynchronize)         \
    X(cuModuleLoadData) X(cuModuleUnload) X(cuModuleGetFunction) X(cuFuncSetAttribute)              \
    X(cuFuncGetAttribute) X(cuOccupancyMaxActiveBlocksPerMultiprocessor) X(cuLaunchKernelEx)        \
    X(cuMemAlloc) X(cuMemFree) X(cuMemsetD8) X(cuMemcpyDtoH) X(cuStreamSynchronize)                 \
    X(cuTensorMapEncodeTiled) X(cuGetErrorString) X(cuOccupancyMaxActiveClusters)                   \
    X(cuStreamGetCaptureInfo) X(cuMemsetD32Async)

struct Driver {
#define X(sym) decltype(&sym) sym##_ = nullptr;
    TK_DRIVER_SYMBOLS(X)
#undef X
    bool ready = false;
};

Driver g_driver;
std::once_flag g_driver_once;
char g_driver_error[256] = "";

void load_driver() {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
        snprintf(g_driver_error, sizeof(g_driver_error), "cannot open libcuda.so.1: %s", dlerror());
        return;
    }
#define X(sym)                                                                                      \
    g_driver.sym##_ = reinterpret_cast<decltype(&sym)>(dlsym(lib, TK_STR(sym)));                    \
    if (!g_driver.sym##_) {                                                                         \
        snprintf(g_driver_error, sizeof(g_driver_error), "libcuda.so.1 lacks %s", TK_STR(sym));     \
        return;                                                                                     \
    }
    TK_DRIVER_SYMBOLS(X)
#undef X
    if (g_driver.cuInit_(0) != CUDA_SUCCESS) {
        snprintf(g_driver_error, sizeof(g_driver_error), "cuInit failed");
        return;
    }
    g_driver.ready = true;
}

int driver() {
    std::call_once(g_driver_once, load_driver);
    return g_driver.ready ? 0 : fail(TK_E_DRIVER, "trainkernel: %s", g_driver_error);
}

int check(CUresult result, const char* what) {
    if (result == CUDA_SUCCESS) return 0;
    const char* text = nullptr;
    g_driver.cuGetErrorString_(result, &text);
    return fail(static_cast<int>(result), "trainkernel: %s failed: %s", what, text ? text : "unknown CUDA error");
}

constexpr int kSyncSlots = 64;        // one barrier word (phase bit + arrival count) per 128-byte line
constexpr int kSyncStride = 128;
constexpr int kStampCount = 256;     // stage stamps | block 0's barrier arrivals | latest arrivals | peer waits + role trace
constexpr int kMapWays = 4;           // encoded tensor maps remembered per map slot
constexpr int kCarriedWord = 8;       // status word that says "values carried over from the previous launch are valid"

struct ContextScope {
    bool pushed = false;
    explicit ContextScope(CUcontext context) { pushed = g_driver.cuCtxPushCurrent_(context) == CUDA_SUCCESS; }
    ~ContextScope() {
        CUcontext ignored;
        if (pushed) g_driver.cuCtxPopCurrent_(&ignored);
    }
};

}  // namespace

struct tk_module {
    CUdevice device = 0;
    CUcontext context = nullptr;
    CUmodule module = nullptr;
    CUfunction function = nullptr;
    int threads = 0;
    size_t dynamic_smem = 0;
    int n_inputs = 0, n_outputs = 0;
    int slots_in = 1, slots_out = 1, slots_maps = 1;
    std::vector<tk_tensor_map_desc> maps;
    CUdeviceptr state = 0;            // sync slots | status words | stage stamps
    std::atomic<uint32_t> next_slot{0};
    std::atomic<uint64_t> timeout_ns{2000000000ull};
    std::atomic<uint32_t> arrivals{0};
    int sm_count = 0;
    int blocks_per_sm = 0;
    int cluster = 1;
    std::atomic<int> cooperative{1};
    std::atomic<int> early_launch{0};  // launch with programmatic stream serialisation (the kernel waits for its predecessor itself)
    // Encoded tensor maps of recent launches, kMapWays per map slot keyed by base address: a caller that
    // cycles through a few resident batches or double buffers (the common case in an eager loop) does not
    // pay for re-encoding them.
    std::mutex map_mutex;
    std::vector<const void*> map_base;       // [slot * kMapWays + way]
    std::vector<CUtensorMap> map_cache;
    std::vector<uint8_t> map_next;           // way to replace next, per slot
    int max_blocks = 0;               // co-resident capacity for the current cluster size
    size_t param_bytes = 0;
    int ordinal = 0;                  // device ordinal the module was loaded on
    std::atomic<size_t> workspace_bytes{0};  // what the kernel's plan needs (0: not recorded)
    std::atomic<uint64_t> launches{0};       // launches issued through this module
    std::atomic<int> faulted{0};      // tk_module_status saw an error; launches are refused until tk_module_reset
    // Base pointers the kernel's vector accesses take to be 16-byte aligned (bit i: input / output i; set once,
    // right after the module is created, before any launch).
    std::vector<uint8_t> aligned_in, aligned_out;
    std::atomic<int> aligned_workspace{0};
    std::atomic<unsigned long long> capture_id{0};   // last stream capture a launch was recorded into

    CUdeviceptr sync_slot(uint32_t i) const { return state + static_cast<size_t>(i) * kSyncStride; }
    CUdeviceptr status() const { return state + static_cast<size_t>(kSyncSlots) * kSyncStride; }
    CUdeviceptr stamps() const { return status() + 128; }
    size_t state_bytes() const { return static_cast<size_t>(kSyncSlots) * kSyncStride + 128 + kStampCount * 8; }
};

extern "C" {

const char* tk_last_error(void) { return g_error; }

uint64_t tk_launch_count(void) { return g_launches.load(); }

int tk_module_load(const void* cubin, size_t cubin_bytes, const char* entry, int device, int threads,
                   size_t dynamic_smem, int n_inputs, int n_outputs, const tk_tensor_map_desc* maps,
                   int n_maps, tk_module** out) {
    if (!cubin || !cubin_bytes || !entry || !out || threads <= 0 || n_inputs < 0 || n_outputs < 0 || n_maps < 0 ||
        (n_maps > 0 && !maps))
        return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_load");
    if (int rc = driver()) return rc;
    tk_module* m = new tk_module();
    m->threads = threads;
    m->ordinal = device;
    m->dynamic_smem = dynamic_smem;
    m->n_inputs = n_inputs;
    m->n_outputs = n_outputs;
    m->slots_in = n_inputs > 0 ? n_inputs : 1;
    m->slots_out = n_outputs > 0 ? n_outputs : 1;
    m->slots_maps = n_maps > 0 ? n_maps : 1;
    m->maps.assign(maps, maps + n_maps);
    m->param_bytes = 128 * static_cast<size_t>(m->slots_maps) + 8 * static_cast<size_t>(m->slots_in + m->slots_out) + 8 * 6;
    int rc = 0;
    do {
        if ((rc = check(g_driver.cuDeviceGet_(&m->device, device), "cuDeviceGet"))) break;
        if ((rc = check(g_driver.cuDevicePrimaryCtxRetain_(&m->context, m->device), "cuDevicePrimaryCtxRetain"))) break;
        ContextScope scope(m->context);
        if ((rc = check(g_driver.cuModuleLoadData_(&m->module, cubin), "cuModuleLoadData"))) break;
        if ((rc = check(g_driver.cuModuleGetFunction_(&m->function, m->module, entry), "cuModuleGetFunction"))) break;
        if (dynamic_smem > 0 &&
            (rc = check(g_driver.cuFuncSetAttribute_(m->function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                                     static_cast<int>(dynamic_smem)), "cuFuncSetAttribute(dynamic shared memory)")))
            break;
        if ((rc = check(g_driver.cuDeviceGetAttribute_(&m->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, m->device), "cuDeviceGetAttribute"))) break;
        if ((rc = check(g_driver.cuOccupancyMaxActiveBlocksPerMultiprocessor_(&m->blocks_per_sm, m->function, threads, dynamic_smem),
                        "cuOccupancyMaxActiveBlocksPerMultiprocessor")))
            break;
        if (m->blocks_per_sm < 1) { rc = fail(TK_E_CAPACITY, "trainkernel: kernel has no resident blocks"); break; }
        m->max_blocks = m->sm_count * m->blocks_per_sm;
        if ((rc = check(g_driver.cuMemAlloc_(&m->state, m->state_bytes()), "cuMemAlloc(kernel state)"))) break;
        if ((rc = check(g_driver.cuMemsetD8_(m->state, 0, m->state_bytes()), "cuMemsetD8(kernel state)"))) break;
    } while (false);
    if (rc) {
        char saved[sizeof(g_error)];
        memcpy(saved, g_error, sizeof(saved));
        tk_module_unload(m);
        memcpy(g_error, saved, sizeof(saved));
        return rc;
    }
    *out = m;
    return 0;
}

void tk_module_unload(tk_module* m) {
    if (!m) return;
    if (m->context) {
        {
            ContextScope scope(m->context);
            if (m->state) g_driver.cuMemFree_(m->state);
            if (m->module) g_driver.cuModuleUnload_(m->module);
        }
        g_driver.cuDevicePrimaryCtxRelease_(m->device);
    }
    delete m;
}

int tk_module_launch(tk_module* m, const void* const* inputs, void* const* outputs, void* workspace, int grid, void* stream) {
    return tk_module_launch_flags(m, inputs, outputs, workspace, grid, stream, 0u);
}

int tk_module_launch_flags(tk_module* m, const void* const* inputs, void* const* outputs, void* workspace, int grid, void* stream,
                           uint32_t flags) {
    if (!m || grid < 1 || (m->n_inputs > 0 && !inputs) || (m->n_outputs > 0 && !outputs))
        return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_launch");
    if (m->faulted.load())
        return fail(TK_E_KERNEL, "trainkernel: an earlier launch of this kernel reported a timed-out wait; call tk_module_reset before launching again");
    if (grid > m->max_blocks || grid % m->cluster)
        return fail(TK_E_CAPACITY, "trainkernel: grid %d exceeds the %d co-resident blocks a cooperative launch allows (cluster size %d)", grid,
                    m->max_blocks, m->cluster);
    // Pointers the kernel reads and writes with 16-byte vector accesses: a misaligned one would fault on the device.
    for (size_t i = 0; i < m->aligned_in.size() && i < static_cast<size_t>(m->n_inputs); ++i)
        if (m->aligned_in[i] && (reinterpret_cast<uintptr_t>(inputs[i]) & 15))
            return fail(TK_E_ARGUMENT, "trainkernel: input %zu is not 16-byte aligned (this kernel was generated for aligned tensors; generate it with assume_aligned=False)", i);
    for (size_t i = 0; i < m->aligned_out.size() && i < static_cast<size_t>(m->n_outputs); ++i)
        if (m->aligned_out[i] && (reinterpret_cast<uintptr_t>(outputs[i]) & 15))
            return fail(TK_E_ARGUMENT, "trainkernel: output %zu is not 16-byte aligned (this kernel was generated for aligned tensors; generate it with assume_aligned=False)", i);
    if (m->aligned_workspace.load() && (reinterpret_cast<uintptr_t>(workspace) & 15))
        return fail(TK_E_ARGUMENT, "trainkernel: the workspace is not 16-byte aligned");
    // Kernel parameter block: tensor maps, input pointers, output pointers, then the scalars.
    alignas(64) unsigned char block[8192];
    if (m->param_bytes > sizeof(block)) return fail(TK_E_ARGUMENT, "trainkernel: parameter block too large");
    memset(block, 0, m->param_bytes);
    for (size_t i = 0; i < m->maps.size(); ++i) {
        const tk_tensor_map_desc& d = m->maps[i];
        const unsigned char* base = nullptr;
        if (d.base_kind == TK_BASE_INPUT && d.base_index >= 0 && d.base_index < m->n_inputs) base = static_cast<const unsigned char*>(inputs[d.base_index]);
        else if (d.base_kind == TK_BASE_OUTPUT && d.base_index >= 0 && d.base_index < m->n_outputs) base = static_cast<const unsigned char*>(outputs[d.base_index]);
        else if (d.base_kind == TK_BASE_WORKSPACE) base = static_cast<const unsigned char*>(workspace);
        if (!base) return fail(TK_E_ARGUMENT, "trainkernel: tensor map %zu has no base pointer", i);
        base += d.byte_offset;
        if (reinterpret_cast<uintptr_t>(base) & 15)
            return fail(TK_E_ARGUMENT, "trainkernel: tensor-core operand %zu is not 16-byte aligned", i);
        std::lock_guard<std::mutex> guard(m->map_mutex);
        if (m->map_base.size() != m->maps.size() * kMapWays) {
            m->map_base.assign(m->maps.size() * kMapWays, nullptr);
            m->map_cache.resize(m->maps.size() * kMapWays);
            m->map_next.assign(m->maps.size(), 0);
        }
        int way = -1;
        for (int w = 0; w < kMapWays; ++w)
            if (m->map_base[i * kMapWays + w] == base) { way = w; break; }
        if (way < 0) {
            way = m->map_next[i];
            m->map_next[i] = static_cast<uint8_t>((way + 1) % kMapWays);
            cuuint64_t dims[2] = {d.inner, d.outer};
            cuuint64_t strides[1] = {d.outer_stride_bytes};
            cuuint32_t box[2] = {d.box_inner, d.box_outer};
            cuuint32_t element_strides[2] = {1, 1};
            m->map_base[i * kMapWays + way] = nullptr;
            CUresult result = g_driver.cuTensorMapEncodeTiled_(
                &m->map_cache[i * kMapWays + way], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                const_cast<unsigned char*>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (int rc = check(result, "cuTensorMapEncodeTiled")) return rc;
            m->map_base[i * kMapWays + way] = base;
        }
        memcpy(block + 128 * i, &m->map_cache[i * kMapWays + way], sizeof(CUtensorMap));
    }
    unsigned char* cursor = block + 128 * static_cast<size_t>(m->slots_maps);
    for (int i = 0; i < m->n_inputs; ++i) memcpy(cursor + 8 * i, &inputs[i], 8);
    cursor += 8 * static_cast<size_t>(m->slots_in);
    for (int i = 0; i < m->n_outputs; ++i) memcpy(cursor + 8 * i, &outputs[i], 8);
    cursor += 8 * static_cast<size_t>(m->slots_out);
    const uint32_t slot = m->next_slot.fetch_add(1) % kSyncSlots;
    const CUdeviceptr sync = m->sync_slot(slot), status = m->status(), stamps = m->stamps();
    const uint64_t timeout = m->timeout_ns.load();
    const uint32_t arrivals = m->arrivals.load();
    memcpy(cursor, &workspace, 8);
    memcpy(cursor + 8, &sync, 8);
    memcpy(cursor + 16, &status, 8);
    memcpy(cursor + 24, &stamps, 8);
    memcpy(cursor + 32, &timeout, 8);
    memcpy(cursor + 40, &arrivals, 4);

    ContextScope scope(m->context);
    // Values carried over from the previous launch are trusted only on the caller's word, and never by the
    // first launch recorded into a stream capture: a replayed graph starts from whatever the caller left.
    if (flags & TK_LAUNCH_TRUST_CARRIED) {
        CUstreamCaptureStatus capture = CU_STREAM_CAPTURE_STATUS_NONE;
        cuuint64_t id = 0;
        if (g_driver.cuStreamGetCaptureInfo_(static_cast<CUstream>(stream), &capture, &id, nullptr, nullptr, nullptr) != CUDA_SUCCESS)
            flags &= ~TK_LAUNCH_TRUST_CARRIED;
        else if (capture == CU_STREAM_CAPTURE_STATUS_ACTIVE && m->capture_id.exchange(id) != id)
            flags &= ~TK_LAUNCH_TRUST_CARRIED;
    }
    memcpy(cursor + 44, &flags, 4);

    CUlaunchAttribute attribute[3];
    memset(attribute, 0, sizeof(attribute));
    unsigned attributes = 0;
    if (m->cooperative.load()) {
        attribute[attributes].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
        attribute[attributes].value.cooperative = 1;
        ++attributes;
    }
    if (m->cluster > 1) {
        attribute[attributes].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attribute[attributes].value.clusterDim.x = static_cast<unsigned>(m->cluster);
        attribute[attributes].value.clusterDim.y = attribute[attributes].value.clusterDim.z = 1;
        ++attributes;
    }
    if (m->early_launch.load()) {
        attribute[attributes].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attribute[attributes].value.programmaticStreamSerializationAllowed = 1;
        ++attributes;
    }
    CUlaunchConfig config;
    memset(&config, 0, sizeof(config));
    config.gridDimX = static_cast<unsigned>(grid);
    config.gridDimY = config.gridDimZ = 1;
    config.blockDimX = static_cast<unsigned>(m->threads);
    config.blockDimY = config.blockDimZ = 1;
    config.sharedMemBytes = static_cast<unsigned>(m->dynamic_smem);
    config.hStream = static_cast<CUstream>(stream);
    config.attrs = attribute;
    config.numAttrs = attributes;
    void* params[1] = {block};
    if (int rc = check(g_driver.cuLaunchKernelEx_(&config, m->function, params, nullptr), "cuLaunchKernelEx")) return rc;
    g_launches.fetch_add(1);
    m->launches.fetch_add(1);
    return 0;
}

int tk_module_resource_usage(tk_module* m, int64_t out[4]) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_resource_usage");
    ContextScope scope(m->context);
    int regs = 0, local = 0, shared = 0;
    if (int rc = check(g_driver.cuFuncGetAttribute_(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, m->function), "cuFuncGetAttribute")) return rc;
    if (int rc = check(g_driver.cuFuncGetAttribute_(&local, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, m->function), "cuFuncGetAttribute")) return rc;
    if (int rc = check(g_driver.cuFuncGetAttribute_(&shared, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, m->function), "cuFuncGetAttribute")) return rc;
    out[0] = regs;
    out[1] = local;
    out[2] = static_cast<int64_t>(shared) + static_cast<int64_t>(m->dynamic_smem);
    out[3] = m->blocks_per_sm;
    return 0;
}

int tk_module_max_coresident_blocks(tk_module* m, int* out) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_max_coresident_blocks");
    *out = m->max_blocks;
    return 0;
}

int tk_module_set_cluster(tk_module* m, int size) {
    if (!m || (size != 1 && size != 2 && size != 4 && size != 8)) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_cluster");
    if (size == 1) {
        m->cluster = 1;
        m->max_blocks = m->sm_count * m->blocks_per_sm;
        return 0;
    }
    ContextScope scope(m->context);
    CUlaunchAttribute attribute;
    memset(&attribute, 0, sizeof(attribute));
    attribute.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attribute.value.clusterDim.x = static_cast<unsigned>(size);
    attribute.value.clusterDim.y = attribute.value.clusterDim.z = 1;
    CUlaunchConfig config;
    memset(&config, 0, sizeof(config));
    config.gridDimX = static_cast<unsigned>(m->sm_count - m->sm_count % size);
    config.gridDimY = config.gridDimZ = 1;
    config.blockDimX = static_cast<unsigned>(m->threads);
    config.blockDimY = config.blockDimZ = 1;
    config.sharedMemBytes = static_cast<unsigned>(m->dynamic_smem);
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (int rc = check(g_driver.cuOccupancyMaxActiveClusters_(&clusters, m->function, &config), "cuOccupancyMaxActiveClusters")) return rc;
    if (clusters < 1) return fail(TK_E_CAPACITY, "trainkernel: no cluster of %d blocks can be resident", size);
    m->cluster = size;
    m->max_blocks = clusters * size;
    return 0;
}

int tk_module_set_cooperative(tk_module* m, int enabled) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_cooperative");
    m->cooperative.store(enabled ? 1 : 0);
    return 0;
}

int tk_module_set_early_launch(tk_module* m, int enabled) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_early_launch");
    m->early_launch.store(enabled ? 1 : 0);
    return 0;
}

int tk_module_status(tk_module* m, void* stream, uint32_t out[4]) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_status");
    ContextScope scope(m->context);
    if (int rc = check(g_driver.cuStreamSynchronize_(static_cast<CUstream>(stream)), "cuStreamSynchronize")) return rc;
    if (int rc = check(g_driver.cuMemcpyDtoH_(out, m->status(), 16), "cuMemcpyDtoH(status)")) return rc;
    if (out[0] != 0) m->faulted.store(1);
    if (out[0] != 0)
        return fail(TK_E_KERNEL, "trainkernel: kernel wait timed out (code %u, stage %u, block %u, detail %u)", out[0], out[1], out[2], out[3]);
    return 0;
}

int tk_module_reset(tk_module* m) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_reset");
    ContextScope scope(m->context);
    if (int rc = check(g_driver.cuCtxSynchronize_(), "cuCtxSynchronize")) return rc;
    if (int rc = check(g_driver.cuMemsetD8_(m->state, 0, m->state_bytes()), "cuMemsetD8(kernel state)")) return rc;
    m->faulted.store(0);
    return 0;
}

int tk_module_device(tk_module* m, int* out) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_device");
    *out = m->ordinal;
    return 0;
}

int tk_module_launches(tk_module* m, uint64_t* out) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_launches");
    *out = m->launches.load();
    return 0;
}

int tk_module_require_alignment(tk_module* m, const uint8_t* inputs, int n_inputs, const uint8_t* outputs, int n_outputs, int workspace) {
    if (!m || n_inputs < 0 || n_outputs < 0 || n_inputs > m->n_inputs || n_outputs > m->n_outputs || (n_inputs && !inputs) || (n_outputs && !outputs))
        return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_require_alignment");
    m->aligned_in.assign(inputs, inputs + n_inputs);
    m->aligned_out.assign(outputs, outputs + n_outputs);
    m->aligned_workspace.store(workspace ? 1 : 0);
    return 0;
}

int tk_module_set_workspace_bytes(tk_module* m, size_t bytes) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_workspace_bytes");
    m->workspace_bytes.store(bytes);
    return 0;
}

int tk_module_workspace_bytes(tk_module* m, size_t* out) {
    if (!m || !out) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_workspace_bytes");
    *out = m->workspace_bytes.load();
    return 0;
}

int tk_module_invalidate_carried(tk_module* m, void* stream) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_invalidate_carried");
    ContextScope scope(m->context);
    return check(g_driver.cuMemsetD32Async_(m->status() + 4 * kCarriedWord, 0u, 1, static_cast<CUstream>(stream)), "cuMemsetD32Async(carried word)");
}

int tk_module_set_timeout(tk_module* m, uint64_t nanoseconds) {
    if (!m || nanoseconds == 0) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_timeout");
    m->timeout_ns.store(nanoseconds);
    return 0;
}

int tk_module_set_expected_arrivals(tk_module* m, uint32_t arrivals) {
    if (!m) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_set_expected_arrivals");
    m->arrivals.store(arrivals);
    return 0;
}

int tk_module_stage_stamps(tk_module* m, void* stream, uint64_t* out, int count) {
    if (!m || !out || count < 0 || count > kStampCount) return fail(TK_E_ARGUMENT, "trainkernel: invalid argument to tk_module_stage_stamps");
    ContextScope scope(m->context);
    if (int rc = check(g_driver.cuStreamSynchronize_(static_cast<CUstream>(stream)), "cuStreamSynchronize")) return rc;
    return check(g_driver.cuMemcpyDtoH_(out, m->stamps(), static_cast<size_t>(count) * 8), "cuMemcpyDtoH(stamps)");
}

}  // extern "C"
