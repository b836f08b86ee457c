// C-ABI of the backend (see include/zen_cuda.h): state, weight residency, uploads and
// kernel launches.  Host logic only; the kernels live in the .cuh files beside it.
//
// The host-pointer calls keep the contract of the reference's GPU backends
// (src/backends/hip/hip_backend.hip:937-1017): lazy latched init, one mutex, weights
// resident by host pointer + shape, synchronous completion.  What differs is deliberate:
// uploads stream through pinned bounce buffers and are re-laid-out on the device, not on
// the host; activations and results cross PCIe through pinned staging; and a declined
// call is an error, because this build has no CPU path to fall back to.
#include "../../include/zen_cuda.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include "decode_ops.cuh"
#include "gemm_q8_0_i8.cuh"
#include "gemm_groups.cuh"
#include "gemv_kq.cuh"
#include "gemv_list.cuh"
#include "gemv_q8_0.cuh"
#include "greedy_pick.cuh"
#include "quantize_acts.cuh"
#include "repack.cuh"
#include "sample_pick.cuh"

struct zen_cuda_gather {
    zk::PeerGather dev{};     // what the kernels receive
    void* counters{};         // local device words: epoch (u64), CTA arrival count (u32), published (u64)
};

struct zen_cuda_gemv_list {
    std::vector<zk::GemvListItem> items;   // they travel as kernel parameters, up to zk::kListMaxItems per launch
    unsigned int* d_counter{};              // device word the CTAs count finished items on (zero between launches)
    uint32_t kpad_blocks{};
    int digits{};
    size_t smem{};
    uint64_t algorithmic_bytes{};  // raw GGUF bytes of all tensors + fp32 inputs and outputs
};

struct zen_cuda_weights {
    int format{};
    size_t rows{}, cols{};
    uint32_t nb{}, nbp{};     // blocks per row, padded to 8
    void* plane[4]{};         // format-specific planes (see repack.cuh)
    void* d_tile_maps{};      // Q8_0 rows of several K segments: zk::GemvTileMaps in device memory (see make_tile_maps), else null
    int kernel_format{};      // what the decode kernel is instantiated for: the format, or zk::kFormatQ6KCodes for Q6_K with unpacked codes
    // Two-digit planes under one scale per 256 weights (gemm_groups.cuh), built at the tensor's first many-row product and
    // kept: wh, wl [rows][cols] int8, units [rows][cols / 256] fp32.
    mutable void* g_hi{};
    mutable void* g_lo{};
    mutable float* g_unit{};
    mutable size_t g_bytes{};
    size_t device_bytes{};
    size_t raw_bytes{};
};

namespace {

using clock_type = std::chrono::steady_clock;
uint64_t us_since(clock_type::time_point t0) {
    return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::microseconds>(clock_type::now() - t0).count());
}

constexpr size_t kBounceBytes = size_t(32) << 20;  // each of the two pinned upload buffers

struct ResidentKey {
    const uint8_t* ptr; size_t rows, cols; int format;
    bool operator==(const ResidentKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && format == o.format; }
};
struct ResidentKeyHash {
    size_t operator()(const ResidentKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<size_t>()(k.rows * 1000003u + k.cols) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h ^ static_cast<size_t>(k.format);
    }
};

struct State {
    std::mutex mutex;
    bool ready{}, failed{};
    int device{};
    int sm_count{};
    int clock_khz{};          // top SM clock, for converting a wait budget in milliseconds into cycles
    size_t smem_optin{};
    cudaStream_t stream{}, copy_stream{};
    cudaEvent_t bounce_free[2]{};
    uint8_t* bounce[2]{};
    zen_cuda_adapter_info adapter{};
    zen_cuda_stats stats{};
    std::string last_error;
    int q8_act_mode{ZEN_CUDA_ACT_INT8};
    bool pdl{true};          // programmatic dependent launch of the GEMV kernels (ZEN_CUDA_PDL=0 turns it off)
    unsigned ctas_per_sm{1}; // persistent GEMV CTAs per SM (ZEN_CUDA_GEMV_CTAS)
    std::unordered_map<ResidentKey, zen_cuda_weights*, ResidentKeyHash> resident;
    bool q6k_codes{true};     // Q6_K tensors keep their codes unpacked on the device (1.07 B per weight for 0.82; ZEN_CUDA_Q6K_CODES=0 keeps ql | qh)
    // Residency budget of the pointer-keyed set (zen::hip keeps weights below 80 % of VRAM, hip_backend.hip:50 and :459-476).
    uint64_t vram_budget{};   // bytes; 0 = no limit
    uint64_t evictions{};     // times the whole keyed set was dropped to make room
    // pinned host staging + device scratch for the host-pointer calls (grow-only)
    float* h_stage{}; size_t h_stage_bytes{};
    float* d_x{}; size_t d_x_bytes{};
    float* d_y{}; size_t d_y_bytes{};
    uint8_t* d_gemm_ws{}; size_t d_gemm_ws_bytes{};  // quantised activations of the prefill GEMM: codes, then block-major scales
    unsigned list_ahead_units{0};   // list launches: row groups of the next item the producer asks L2 for at an item boundary (ZEN_CUDA_LIST_AHEAD; measured: no gain, default off)
    bool warm_hints{true};    // honour zen_cuda_gemv_fusion.warm_next (ZEN_CUDA_WARM=0 ignores the hints)
    bool gemm_stream_k{true}; // prefill GEMM: even K-tile shares when tiles do not divide the SMs (ZEN_CUDA_GEMM_STREAMK=0 turns it off)
    bool use_gemm{true};     // tensor-core prefill path (ZEN_CUDA_GEMM=0 falls back to chunks of eight tokens on the decode kernel)
    bool gemm_groups{true};  // Q8_0 many-row products through the group-scale kernel (ZEN_CUDA_GEMM_GROUPS=0: the per-block kernel)
    void* encode_tiled{};    // cuTensorMapEncodeTiled, resolved through the runtime
    int* h_error{};   // mapped pinned word the kernels write on a bounded-wait timeout
    int* d_error{};   // device alias of h_error
    // Small results skip the copy engine: the kernels store them straight into mapped pinned memory, a one-thread
    // kernel behind them raises a sequence number there, and the calling thread polls it.
    float* h_result{}; float* d_result{}; size_t h_result_bytes{};
    float* h_input{}; float* d_input{};   // mapped pinned staging for small activations, read by stage_in_kernel
    volatile unsigned* h_done{}; unsigned* d_done{}; unsigned done_seq{};
    unsigned* d_seq{};        // device word: number of results published so far (the copy-out kernel counts, so a captured launch can be replayed)
    // Host-pointer calls that are one product launch long are replayed from a captured graph (fetch -> product -> copy-out):
    // one cudaGraphLaunch instead of three kernel launches per call.  Keyed by the resident tensors and the call's shape;
    // dropped whenever a pointer inside could have changed (scratch regrown, a tensor released, shutdown).
    struct HostGraph { cudaGraphExec_t exec{}; };
    std::unordered_map<uint64_t, HostGraph> host_graphs;
    bool use_host_graphs{true};   // ZEN_CUDA_HOST_GRAPHS=0 turns the replay off
};

State& state() { static State s; return s; }

bool set_error(State& s, const std::string& msg) {
    s.last_error = msg;
    ++s.stats.fallbacks;
    return false;
}
#define ZC_CUDA(s, call)                                                                                  \
    do {                                                                                                  \
        const cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess) return set_error((s), std::string(#call) + ": " + cudaGetErrorString(e_)); \
    } while (0)

bool opted_out() {
    static const bool out = [] {
        if (const char* b = std::getenv("ZEN_BACKEND")) {
            std::string n(b);
            for (char& c : n) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
            if (!n.empty() && n != "cuda" && n != "gpu" && n != "b200") return true;
        }
        const char* f = std::getenv("ZEN_CUDA");
        return f && f[0] == '0';
    }();
    return out;
}

// Bounded device waits give up after this many milliseconds (converted with the top SM clock; 0 restores the default).
bool apply_wait_budget(State& s, unsigned ms) {
    const long long cycles = ms ? static_cast<long long>(ms) * std::max(1, s.clock_khz) : zk::kDefaultWaitBudgetCycles;
    ZC_CUDA(s, cudaMemcpyToSymbol(zk::g_wait_budget_cycles, &cycles, sizeof cycles));
    return true;
}

bool warm_noalloc_path(State& s);   // defined with the allocation-free entry point

uint64_t default_vram_budget(const State& s);
bool init_locked(State& s) {
    if (s.ready) {
        // Entry points may be reached from any thread, and a new thread starts on device 0: make the backend's device
        // current before anything allocates or launches on its behalf.
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != s.device) {
            if (cudaSetDevice(s.device) != cudaSuccess) return set_error(s, "cudaSetDevice to the backend's device failed");
        }
        return true;
    }
    if (s.failed) return false;
    auto fail = [&s](const std::string& why) { s.failed = true; s.last_error = why; return false; };
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) return fail("no CUDA device");
    int dev = 0;
    if (const char* lr = std::getenv("LOCAL_RANK")) dev = std::atoi(lr) % n;   // one process per GPU
    if (const char* d = std::getenv("ZEN_CUDA_DEVICE")) dev = std::atoi(d) % n;
    if (cudaSetDevice(dev) != cudaSuccess) return fail("cudaSetDevice failed");
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fail("cudaGetDeviceProperties failed");
    if (prop.major != 10) return fail(std::string("device is sm_") + std::to_string(prop.major * 10 + prop.minor) + ", this build is sm_100a only");
    s.device = dev;
    s.sm_count = prop.multiProcessorCount;
    s.smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaDeviceGetAttribute(&s.clock_khz, cudaDevAttrClockRate, dev) != cudaSuccess) s.clock_khz = 1965000;
    std::snprintf(s.adapter.name, sizeof(s.adapter.name), "%.127s", prop.name);
    s.adapter.dedicated_vram = prop.totalGlobalMem;
    s.vram_budget = default_vram_budget(s);
    if (const char* m = std::getenv("ZEN_CUDA_VRAM_BUDGET_MB")) s.vram_budget = static_cast<uint64_t>(std::max(0ll, std::atoll(m))) << 20;
    s.adapter.shared_memory = prop.sharedMemPerBlockOptin;
    s.adapter.sm_count = prop.multiProcessorCount;
    s.adapter.warp_size = prop.warpSize;
    std::snprintf(s.adapter.arch, sizeof(s.adapter.arch), "sm_%d", prop.major * 10 + prop.minor);
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return fail("stream create failed");
    if (cudaStreamCreateWithFlags(&s.copy_stream, cudaStreamNonBlocking) != cudaSuccess) return fail("stream create failed");
    for (int i = 0; i < 2; ++i) {
        if (cudaEventCreateWithFlags(&s.bounce_free[i], cudaEventDisableTiming) != cudaSuccess) return fail("event create failed");
        if (cudaHostAlloc(reinterpret_cast<void**>(&s.bounce[i]), kBounceBytes, cudaHostAllocDefault) != cudaSuccess) return fail("pinned alloc failed");
    }
    if (cudaHostAlloc(reinterpret_cast<void**>(&s.h_error), sizeof(int), cudaHostAllocMapped) != cudaSuccess) return fail("pinned alloc failed");
    *s.h_error = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.d_error), s.h_error, 0) != cudaSuccess) return fail("mapped pointer failed");
    if (const char* m = std::getenv("ZEN_CUDA_Q8_ACT")) {
        if (!std::strcmp(m, "fp32") || !std::strcmp(m, "2")) s.q8_act_mode = ZEN_CUDA_ACT_FP32;
        else if (!std::strcmp(m, "int8") || !std::strcmp(m, "1")) s.q8_act_mode = ZEN_CUDA_ACT_INT8;
    }
    if (const char* m = std::getenv("ZEN_CUDA_PDL")) s.pdl = m[0] != '0';
    if (const char* m = std::getenv("ZEN_CUDA_GEMM")) s.use_gemm = m[0] != '0';
    if (const char* m = std::getenv("ZEN_CUDA_GEMM_GROUPS")) s.gemm_groups = m[0] != '0';
    if (const char* m = std::getenv("ZEN_CUDA_GEMM_STREAMK")) s.gemm_stream_k = m[0] != '0';
    if (const char* m = std::getenv("ZEN_CUDA_WARM")) s.warm_hints = m[0] != '0';
    if (const char* m = std::getenv("ZEN_CUDA_HOST_GRAPHS")) s.use_host_graphs = m[0] != '0';
    {
        cudaDriverEntryPointQueryResult qres{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &s.encode_tiled, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            s.encode_tiled = nullptr;
    }
    if (const char* m = std::getenv("ZEN_CUDA_Q6K_CODES")) s.q6k_codes = std::atoi(m) != 0;
    if (const char* m = std::getenv("ZEN_CUDA_GEMV_CTAS")) s.ctas_per_sm = static_cast<unsigned>(std::max(1, std::min(4, std::atoi(m))));
    if (const char* m = std::getenv("ZEN_CUDA_LIST_AHEAD")) s.list_ahead_units = static_cast<unsigned>(std::max(0, std::min(64, std::atoi(m))));
    if (const char* m = std::getenv("ZEN_CUDA_WAIT_MS")) {
        if (!apply_wait_budget(s, static_cast<unsigned>(std::max(0, std::atoi(m))))) return fail("setting the wait budget failed");
    }
    // Everything the allocation-free entry point needs that may itself allocate (module loading, the scratch array's
    // address, the GEMM's shared-memory opt-in) happens here, where allocating is allowed.
    if (!warm_noalloc_path(s)) return fail("preparing the allocation-free GEMM path failed: " + s.last_error);
    s.ready = true;
    return true;
}

// zen::hip's kVRAMBudgetPercent (hip_backend.hip:50): resident weights stay below 80 % of the device's memory.
uint64_t default_vram_budget(const State& s) { return s.adapter.dedicated_vram / 100 * 80; }

void free_weights(State& s, zen_cuda_weights* w) {
    if (!w) return;
    for (void* p : w->plane) if (p) cudaFree(p);
    if (w->d_tile_maps) cudaFree(w->d_tile_maps);
    if (w->g_hi) cudaFree(w->g_hi);
    if (w->g_lo) cudaFree(w->g_lo);
    if (w->g_unit) cudaFree(w->g_unit);
    s.stats.weight_bytes -= std::min<uint64_t>(s.stats.weight_bytes, w->device_bytes + w->g_bytes);
    delete w;
}

bool super_block_format(int fmt) { return fmt == ZEN_CUDA_Q6_K || fmt == ZEN_CUDA_Q4_K || fmt == ZEN_CUDA_Q5_K; }
uint32_t block_elems(int fmt) { return super_block_format(fmt) ? 256u : 32u; }
int plane_count(int fmt) { return fmt == ZEN_CUDA_Q8_0 || fmt == ZEN_CUDA_Q4_0 ? 2 : fmt == ZEN_CUDA_Q4_K ? 3 : 4; }
uint32_t block_bytes(int fmt) {
    return fmt == ZEN_CUDA_Q8_0 ? 34u : fmt == ZEN_CUDA_Q4_0 ? 18u : fmt == ZEN_CUDA_Q6_K ? 210u : fmt == ZEN_CUDA_Q4_K ? 144u : fmt == ZEN_CUDA_Q5_K ? 176u : 0u;
}

// Streams [src, src+bytes) to `dst` on the copy stream through the two pinned bounce buffers:
// the CPU fills one while the DMA engine drains the other.
bool stream_to_device(State& s, void* dst, const uint8_t* src, size_t bytes) {
    size_t off = 0;
    int which = 0;
    while (off < bytes) {
        const size_t n = std::min(kBounceBytes, bytes - off);
        ZC_CUDA(s, cudaEventSynchronize(s.bounce_free[which]));
        const auto t0 = clock_type::now();
        std::memcpy(s.bounce[which], src + off, n);
        s.stats.stage_us += us_since(t0);
        ZC_CUDA(s, cudaMemcpyAsync(static_cast<uint8_t*>(dst) + off, s.bounce[which], n, cudaMemcpyHostToDevice, s.copy_stream));
        ZC_CUDA(s, cudaEventRecord(s.bounce_free[which], s.copy_stream));
        off += n;
        which ^= 1;
    }
    return true;
}

// Device bytes of each plane of a tensor; every plane gets slack for bulk copies whose size was rounded up to 16 bytes.
void plane_sizes(int fmt, size_t nrows, size_t cols, size_t plane_bytes[4], bool q6k_codes) {
    const uint32_t nb = static_cast<uint32_t>(cols / block_elems(fmt)), nbp = (nb + 7u) & ~7u;
    plane_bytes[0] = plane_bytes[1] = plane_bytes[2] = plane_bytes[3] = 0;
    if (fmt == ZEN_CUDA_Q4_K || fmt == ZEN_CUDA_Q5_K) {   // nb counts 256-weight super-blocks
        int i = 0;
        plane_bytes[i++] = nrows * (cols / 2) + 64;                        // nibbles
        if (fmt == ZEN_CUDA_Q5_K) plane_bytes[i++] = nrows * (cols / 8) + 64;   // fifth bits
        plane_bytes[i++] = nrows * (cols / 16) + 64;                       // unpacked sub-block scales | minimums
        plane_bytes[i++] = nrows * static_cast<size_t>(nbp) * 4 + 64;      // (d, dmin) f16 pairs
    } else if (fmt == ZEN_CUDA_Q8_0) {
        plane_bytes[0] = nrows * cols + 64;                                // int8 codes
        plane_bytes[1] = nrows * static_cast<size_t>(nbp) * 2 + 64;        // f16 scales
    } else if (fmt == ZEN_CUDA_Q4_0) {
        plane_bytes[0] = nrows * (cols / 2) + 64;                          // nibble bytes
        plane_bytes[1] = nrows * static_cast<size_t>(nbp) * 2 + 64;        // f16 scales
    } else if (q6k_codes) {   // Q6_K, codes unpacked
        plane_bytes[0] = nrows * cols + 64;                                // q - 32, int8
        plane_bytes[1] = nrows * (cols / 16) + 64;                         // int8 group scales
        plane_bytes[2] = nrows * static_cast<size_t>(nbp) * 2 + 64;        // f16 super-block scales
    } else {  // Q6_K: nb counts 256-weight super-blocks
        plane_bytes[0] = nrows * (cols / 2) + 64;                          // ql
        plane_bytes[1] = nrows * (cols / 4) + 64;                          // qh
        plane_bytes[2] = nrows * (cols / 16) + 64;                         // int8 group scales
        plane_bytes[3] = nrows * static_cast<size_t>(nbp) * 2 + 64;        // f16 super-block scales
    }
}

bool make_tile_maps(State& s, zen_cuda_weights* w);   // defined with the other tensor-map code below
bool make_kq_tile_maps(State& s, zen_cuda_weights* w);

// Uploads rows [first_row, first_row+nrows) and re-lays them out into planes on the device.
zen_cuda_weights* upload_locked(State& s, int fmt, const uint8_t* host, size_t rows_total, size_t cols, size_t first_row, size_t nrows) {
    const uint32_t be = block_elems(fmt), bb = block_bytes(fmt);
    if (!bb || !host || !nrows || !cols || cols % be || first_row + nrows > rows_total) {
        set_error(s, "upload: bad shape or format");
        return nullptr;
    }
    const auto t_all = clock_type::now();
    auto* w = new zen_cuda_weights;
    w->format = fmt; w->rows = nrows; w->cols = cols;
    w->nb = static_cast<uint32_t>(cols / be);
    w->nbp = (w->nb + 7u) & ~7u;
    const size_t row_raw = static_cast<size_t>(w->nb) * bb;
    w->raw_bytes = nrows * row_raw;
    uint8_t* d_raw = nullptr;
    auto t0 = clock_type::now();
    bool ok = cudaMalloc(reinterpret_cast<void**>(&d_raw), w->raw_bytes + 16) == cudaSuccess;
    size_t plane_bytes[4];
    const bool codes_layout = fmt == ZEN_CUDA_Q6_K && s.q6k_codes;
    w->kernel_format = codes_layout ? zk::kFormatQ6KCodes : fmt;
    plane_sizes(fmt, nrows, cols, plane_bytes, s.q6k_codes);
    for (int i = 0; ok && i < 4; ++i)
        if (plane_bytes[i]) {
            ok = cudaMalloc(&w->plane[i], plane_bytes[i]) == cudaSuccess;
            if (ok) { ok = cudaMemsetAsync(w->plane[i], 0, plane_bytes[i], s.copy_stream) == cudaSuccess; w->device_bytes += plane_bytes[i]; }
        }
    s.stats.alloc_us += us_since(t0);
    if (!ok) {
        set_error(s, std::string("upload: device allocation failed: ") + cudaGetErrorString(cudaGetLastError()));
        if (d_raw) cudaFree(d_raw);
        for (void* p : w->plane) if (p) cudaFree(p);
        delete w;
        return nullptr;
    }
    t0 = clock_type::now();
    ok = stream_to_device(s, d_raw, host + first_row * row_raw, w->raw_bytes);
    s.stats.transfer_us += us_since(t0);
    if (ok) {
        t0 = clock_type::now();
        const size_t nblocks = nrows * w->nb;
        const unsigned grid = static_cast<unsigned>((nblocks + 255) / 256);
        if (fmt == ZEN_CUDA_Q8_0)
            zk::repack_q8_0_kernel<<<grid, 256, 0, s.copy_stream>>>(d_raw, static_cast<uint8_t*>(w->plane[0]),
                                                                   static_cast<uint16_t*>(w->plane[1]), nrows, w->nb, w->nbp);
        else if (fmt == ZEN_CUDA_Q4_0)
            zk::repack_q4_0_kernel<<<grid, 256, 0, s.copy_stream>>>(d_raw, static_cast<uint8_t*>(w->plane[0]),
                                                                   static_cast<uint16_t*>(w->plane[1]), nrows, w->nb, w->nbp);
        else if (fmt == ZEN_CUDA_Q4_K)
            zk::repack_k45_kernel<false><<<grid, 256, 0, s.copy_stream>>>(d_raw, static_cast<uint8_t*>(w->plane[0]), nullptr, static_cast<uint8_t*>(w->plane[1]),
                                                                         static_cast<uint32_t*>(w->plane[2]), nrows, w->nb, w->nbp);
        else if (fmt == ZEN_CUDA_Q5_K)
            zk::repack_k45_kernel<true><<<grid, 256, 0, s.copy_stream>>>(d_raw, static_cast<uint8_t*>(w->plane[0]), static_cast<uint8_t*>(w->plane[1]),
                                                                        static_cast<uint8_t*>(w->plane[2]), static_cast<uint32_t*>(w->plane[3]), nrows, w->nb, w->nbp);
        else if (codes_layout)
            zk::unpack_q6_k_codes_kernel<<<static_cast<unsigned>((nblocks * 16 + 255) / 256), 256, 0, s.copy_stream>>>(
                d_raw, static_cast<int8_t*>(w->plane[0]), static_cast<int8_t*>(w->plane[1]), static_cast<uint16_t*>(w->plane[2]), nrows, w->nb, w->nbp);
        else
            zk::repack_q6_k_kernel<<<grid, 256, 0, s.copy_stream>>>(d_raw, static_cast<uint8_t*>(w->plane[0]), static_cast<uint8_t*>(w->plane[1]),
                                                                   static_cast<int8_t*>(w->plane[2]), static_cast<uint16_t*>(w->plane[3]),
                                                                   nrows, w->nb, w->nbp);
        ++s.stats.dispatches;
        ok = cudaGetLastError() == cudaSuccess && cudaStreamSynchronize(s.copy_stream) == cudaSuccess;
        s.stats.repack_us += us_since(t0);
        if (!ok) set_error(s, "upload: repack failed");
    }
    if (d_raw) cudaFree(d_raw);
    if (!ok) {
        for (void* p : w->plane) if (p) cudaFree(p);
        delete w;
        return nullptr;
    }
    if (!(fmt == ZEN_CUDA_Q8_0 ? make_tile_maps(s, w) : make_kq_tile_maps(s, w))) {
        for (void* p : w->plane) if (p) cudaFree(p);
        delete w;
        return nullptr;
    }
    s.stats.upload_bytes += w->raw_bytes;
    s.stats.weight_bytes += w->device_bytes;
    s.stats.upload_us += us_since(t_all);
    return w;
}

void drop_host_graphs(State& s);   // defined below

// Frees the whole pointer-keyed set.  The reference evicts everything rather than a part (hip_backend.hip:462-471: the
// loader asks for tensors in the same order every run, so a partial eviction would only churn).  Tensors uploaded through
// zen_cuda_dev_upload belong to their caller and stay.
void evict_resident_locked(State& s) {
    cudaStreamSynchronize(s.stream);   // nothing queued may still read them
    drop_host_graphs(s);               // captured calls name their addresses
    for (auto& kv : s.resident) free_weights(s, kv.second);
    s.resident.clear();
    ++s.evictions;
}

zen_cuda_weights* lookup_locked(State& s, int fmt, const uint8_t* host, size_t rows, size_t cols) {
    const ResidentKey key{host, rows, cols, fmt};
    auto it = s.resident.find(key);
    if (it != s.resident.end()) return it->second;
    if (s.vram_budget && block_bytes(fmt) && cols && cols % block_elems(fmt) == 0) {
        size_t pb[4];
        plane_sizes(fmt, rows, cols, pb, s.q6k_codes);
        const uint64_t need = pb[0] + pb[1] + pb[2] + pb[3];
        if (s.stats.weight_bytes + need > s.vram_budget && !s.resident.empty()) evict_resident_locked(s);
        if (s.stats.weight_bytes + need > s.vram_budget) {
            set_error(s, "upload: the tensor does not fit the residency budget");
            return nullptr;
        }
    }
    zen_cuda_weights* w = upload_locked(s, fmt, host, rows, cols, 0, rows);
    if (w) s.resident.emplace(key, w);
    return w;
}

#ifdef ZK_TRACE
unsigned long long* g_trace = nullptr;  // profiling builds: device buffer [launch][148][8]
size_t g_trace_launch = 0;
#endif

template <int kBatch, int kDigits, bool kFuse>
cudaError_t launch_gemv_q8_0(const zk::GemvParams& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    auto* fn = &zk::gemv_q8_0_kernel<kBatch, kDigits, kFuse>;
    static size_t configured = 0;  // per instantiation; one device per process, calls serialised by the backend mutex
    if (smem > configured) {       // raised outside any stream capture by the first (uncaptured) launch of a shape
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        // The kernels stream through shared memory and barely use L1: give shared memory the whole array, so that a
        // CTA of the next launch can become resident beside one of this launch whenever two fit.
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(zk::kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, fn, p);
}

template <int kDigits, bool kFuse>
cudaError_t dispatch_batch_fuse(int batch, const zk::GemvParams& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    switch (batch) {
    case 1: return launch_gemv_q8_0<1, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 2: return launch_gemv_q8_0<2, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 3: return launch_gemv_q8_0<3, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 4: return launch_gemv_q8_0<4, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 5: return launch_gemv_q8_0<5, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 6: return launch_gemv_q8_0<6, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 7: return launch_gemv_q8_0<7, kDigits, kFuse>(p, grid, smem, st, pdl);
    case 8: return launch_gemv_q8_0<8, kDigits, kFuse>(p, grid, smem, st, pdl);
    default: return cudaErrorInvalidValue;
    }
}
// Launches that carry fused work (p.flags) take the kFuse instantiation; plain products keep the lean one.
template <int kDigits>
cudaError_t dispatch_batch(int batch, const zk::GemvParams& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    return (p.flags & ~zk::kGemvFlagWarm) ? dispatch_batch_fuse<kDigits, true>(batch, p, grid, smem, st, pdl)
                                          : dispatch_batch_fuse<kDigits, false>(batch, p, grid, smem, st, pdl);
}

template <int kFormat, int kBatch>
cudaError_t launch_gemv_kq(const zk::KqParams& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    auto* fn = &zk::gemv_kq_kernel<kFormat, kBatch>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        // The kernels stream through shared memory and barely use L1: give shared memory the whole array, so that a
        // CTA of the next launch can become resident beside one of this launch whenever two fit.
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(zk::kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, fn, p);
}

template <int kFormat>
cudaError_t dispatch_kq(int batch, const zk::KqParams& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    switch (batch) {
    case 1: return launch_gemv_kq<kFormat, 1>(p, grid, smem, st, pdl);
    case 2: return launch_gemv_kq<kFormat, 2>(p, grid, smem, st, pdl);
    case 3: return launch_gemv_kq<kFormat, 3>(p, grid, smem, st, pdl);
    case 4: return launch_gemv_kq<kFormat, 4>(p, grid, smem, st, pdl);
    case 5: return launch_gemv_kq<kFormat, 5>(p, grid, smem, st, pdl);
    case 6: return launch_gemv_kq<kFormat, 6>(p, grid, smem, st, pdl);
    case 7: return launch_gemv_kq<kFormat, 7>(p, grid, smem, st, pdl);
    case 8: return launch_gemv_kq<kFormat, 8>(p, grid, smem, st, pdl);
    default: return cudaErrorInvalidValue;
    }
}

size_t gemv_smem_bytes(int format, size_t cols, size_t tokens, int act_mode) {   // format: a kernel format (zen_cuda_weights::kernel_format)
    if (format == ZEN_CUDA_Q8_0) {
        const uint32_t nb = static_cast<uint32_t>(cols / 32), nseg = (nb + zk::kGemvSegBlocks - 1) / zk::kGemvSegBlocks;
        return zk::gemv_q8_0_smem_bytes(nseg, static_cast<int>(tokens), act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1);
    }
    const uint32_t nseg = static_cast<uint32_t>((cols + zk::kKqSegElems - 1) / zk::kKqSegElems);
    return format == ZEN_CUDA_Q4_0   ? zk::gemv_kq_smem_bytes<ZEN_CUDA_Q4_0>(nseg, static_cast<int>(tokens))
           : format == ZEN_CUDA_Q4_K ? zk::gemv_kq_smem_bytes<ZEN_CUDA_Q4_K>(nseg, static_cast<int>(tokens))
           : format == ZEN_CUDA_Q5_K ? zk::gemv_kq_smem_bytes<ZEN_CUDA_Q5_K>(nseg, static_cast<int>(tokens))
           : format == zk::kFormatQ6KCodes ? zk::gemv_kq_smem_bytes<zk::kFormatQ6KCodes>(nseg, static_cast<int>(tokens))
                                     : zk::gemv_kq_smem_bytes<ZEN_CUDA_Q6_K>(nseg, static_cast<int>(tokens));
}

// Largest number of activation rows (<= 8) one launch can keep in shared memory beside the weight ring; 0 if not even one.
size_t max_tokens_per_launch(const State& s, int format, size_t cols, int act_mode) {
    for (size_t t = 8; t >= 1; --t)
        if (gemv_smem_bytes(format, cols, t, act_mode) <= s.smem_optin) return t;
    return 0;
}

bool enqueue_gemv_kq(State& s, const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x,
                     size_t tokens, cudaStream_t st, const zk::PeerGather* gather) {
    zk::KqParams p{};
    if (gather) p.gather = *gather;
    uint32_t total_rows = 0;
    const int fmt = w[0]->kernel_format;
    const int planes = fmt == zk::kFormatQ6KCodes ? 3 : plane_count(fmt);
    for (size_t i = 0; i < count; ++i) {
        for (int k = 0; k < planes; ++k) p.task[i].plane[k] = static_cast<const uint8_t*>(w[i]->plane[k]);
        p.tile_maps[i] = static_cast<const zk::KqTileMaps*>(w[i]->d_tile_maps);
        p.task[i].y = d_y ? d_y[i] : nullptr;
        p.task[i].rows = static_cast<uint32_t>(w[i]->rows);
        p.task[i].first_row = total_rows;
        total_rows += static_cast<uint32_t>(w[i]->rows);
    }
    p.ntasks = static_cast<uint32_t>(count);
    p.total_rows = total_rows;
    p.x = d_x;
    p.K = static_cast<uint32_t>(w[0]->cols);
    p.nseg = (p.K + zk::kKqSegElems - 1) / zk::kKqSegElems;
    if (fmt == ZEN_CUDA_Q4_0) {
        p.pitch[0] = p.K / 2;
        p.pitch[1] = w[0]->nbp * 2;
    } else if (fmt == ZEN_CUDA_Q4_K) {
        p.pitch[0] = p.K / 2; p.pitch[1] = p.K / 16; p.pitch[2] = w[0]->nbp * 4;
    } else if (fmt == ZEN_CUDA_Q5_K) {
        p.pitch[0] = p.K / 2; p.pitch[1] = p.K / 8; p.pitch[2] = p.K / 16; p.pitch[3] = w[0]->nbp * 4;
    } else if (fmt == zk::kFormatQ6KCodes) {
        p.pitch[0] = p.K; p.pitch[1] = p.K / 16; p.pitch[2] = w[0]->nbp * 2;
    } else {
        p.pitch[0] = p.K / 2; p.pitch[1] = p.K / 4; p.pitch[2] = p.K / 16; p.pitch[3] = w[0]->nbp * 2;
    }
    p.error_word = s.d_error;
    const unsigned grid = gather ? gather->grid
                                 : std::max(1u, std::min<unsigned>((total_rows + zk::kGemvWarps - 1) / zk::kGemvWarps, static_cast<unsigned>(s.sm_count)));
    const size_t smem = gemv_smem_bytes(fmt, w[0]->cols, tokens, ZEN_CUDA_ACT_FP32)
                        + (gather ? zk::gather_stash_bytes(total_rows, grid, static_cast<int>(tokens)) : 0);
    if (smem > s.smem_optin) return set_error(s, "gemv: activation rows do not fit shared memory (columns x tokens too large)");
    const cudaError_t e = fmt == ZEN_CUDA_Q4_0   ? dispatch_kq<ZEN_CUDA_Q4_0>(static_cast<int>(tokens), p, grid, smem, st, s.pdl)
                          : fmt == ZEN_CUDA_Q4_K ? dispatch_kq<ZEN_CUDA_Q4_K>(static_cast<int>(tokens), p, grid, smem, st, s.pdl)
                          : fmt == ZEN_CUDA_Q5_K ? dispatch_kq<ZEN_CUDA_Q5_K>(static_cast<int>(tokens), p, grid, smem, st, s.pdl)
                          : fmt == zk::kFormatQ6KCodes ? dispatch_kq<zk::kFormatQ6KCodes>(static_cast<int>(tokens), p, grid, smem, st, s.pdl)
                                                 : dispatch_kq<ZEN_CUDA_Q6_K>(static_cast<int>(tokens), p, grid, smem, st, s.pdl);
    if (e != cudaSuccess) return set_error(s, std::string("gemv launch: ") + cudaGetErrorString(e));
    ++s.stats.dispatches;
    return true;
}

// Enqueues one batched GEMV launch: `count` tensors (same format, same K) times `tokens` (<= 8)
// activation rows.  Device pointers throughout.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(State& s, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args);   // defined below

bool enqueue_gemv(State& s, const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x,
                  size_t tokens, int act_mode, cudaStream_t st, const zk::PeerGather* gather = nullptr, const float* d_gate = nullptr,
                  const float* d_norm_weight = nullptr, float norm_eps = 0.0f, bool accumulate = false, const zen_cuda_weights* warm_next = nullptr,
                  bool swiglu_pair = false) {
    if (!count || count > zk::kMaxTasks || !tokens || tokens > 8 || (!d_x && !gather)) return set_error(s, "gemv: bad batch");
    if (act_mode != ZEN_CUDA_ACT_INT8 && act_mode != ZEN_CUDA_ACT_FP32) return set_error(s, "gemv: bad activation mode");
    zk::GemvParams p{};
    uint32_t total_rows = 0;
    for (size_t i = 0; i < count; ++i) {
        const bool has_y = d_y && d_y[i];
        if (!w[i] || (!has_y && !gather && !(swiglu_pair && i == 1)) || w[i]->format != w[0]->format || w[i]->kernel_format != w[0]->kernel_format ||
            w[i]->cols != w[0]->cols)
            return set_error(s, "gemv: tasks must share format and columns");
        p.task[i].codes = static_cast<const uint8_t*>(w[i]->plane[0]);
        p.task[i].scales = static_cast<const __half*>(w[i]->plane[1]);
        p.tile_maps[i] = static_cast<const zk::GemvTileMaps*>(w[i]->d_tile_maps);
        p.task[i].y = has_y ? d_y[i] : nullptr;
        p.task[i].rows = static_cast<uint32_t>(w[i]->rows);
        p.task[i].first_row = total_rows;
        total_rows += static_cast<uint32_t>(w[i]->rows);
    }
    if (gather) {
        if (tokens * total_rows > gather->slot_floats) return set_error(s, "gemv gather: tokens x rows exceed the gather slot");
        if (!d_x && (tokens != 1 || w[0]->cols != static_cast<size_t>(gather->world) * gather->slot_floats))
            return set_error(s, "gemv gather: a chained input needs one token and columns == world x slot_floats");
        p.gather = *gather;
    }
    if (w[0]->format != ZEN_CUDA_Q8_0) {
        if (act_mode != ZEN_CUDA_ACT_FP32) return set_error(s, "gemv: Q4_0, Q6_K, Q4_K and Q5_K take fp32-equivalent activations only");
        if (d_gate || d_norm_weight || accumulate || swiglu_pair) return set_error(s, "gemv: fused inputs, outputs and accumulation are Q8_0 paths");
        return enqueue_gemv_kq(s, w, d_y, count, d_x, tokens, st, gather);   // a warm_next hint is not used by these kernels (measured: no gain)
    }
    if (d_gate && d_norm_weight) return set_error(s, "gemv: a fused input is either SwiGLU or RMSNorm");
    if (swiglu_pair) {
        // gate and up as one row space: the two teams of a CTA compute row r of both, task 0's output gets silu(g) * u
        if (count != 2 || w[0]->rows != w[1]->rows || gather || accumulate || !d_y || !d_y[0])
            return set_error(s, "gemv: a SwiGLU pair is two tensors of equal shape with an output for the first, without gather or accumulation");
        p.flags |= zk::kGemvFlagPairSwiglu;
        p.task[1].first_row = 0;
        total_rows = static_cast<uint32_t>(w[0]->rows);
    }
    if (d_gate) { p.flags |= zk::kGemvFlagSwiglu; p.x_gate = d_gate; }
    if (d_norm_weight) { p.flags |= zk::kGemvFlagNorm; p.norm_weight = d_norm_weight; p.norm_eps = norm_eps; }
    if (accumulate) p.flags |= zk::kGemvFlagAccumulate;
    // A hint, honoured where it pays: a launch that streams more than kWarmMaxLaunchBytes keeps HBM busy by itself, and a
    // prefetch for its successor then only competes with it (measured: -0.5 us for a 26.8 MB launch, +1.2 us for 62 MB).
    constexpr size_t kWarmMaxLaunchBytes = size_t(32) << 20;
    if (s.warm_hints && warm_next && warm_next->format == ZEN_CUDA_Q8_0 && static_cast<size_t>(total_rows) * w[0]->cols <= kWarmMaxLaunchBytes) {
        p.flags |= zk::kGemvFlagWarm;
        p.warm_codes = static_cast<const uint8_t*>(warm_next->plane[0]);
        p.warm_scales = static_cast<const __half*>(warm_next->plane[1]);
        p.warm_rows = static_cast<uint32_t>(warm_next->rows);
        p.warm_K = static_cast<uint32_t>(warm_next->cols);
        p.warm_nbp = warm_next->nbp;
    }
    p.ntasks = static_cast<uint32_t>(count);
    p.total_rows = total_rows;
    p.x = d_x;
    p.K = static_cast<uint32_t>(w[0]->cols);
    const uint32_t nb = p.K / 32, nseg = (nb + zk::kGemvSegBlocks - 1) / zk::kGemvSegBlocks;
    if (w[0]->nb != nb || w[0]->nbp != ((nb + 7) & ~7u)) return set_error(s, "gemv: resident tensor has an unexpected scale pitch");
    p.error_word = s.d_error;
#ifdef ZK_TRACE
    p.trace = g_trace ? g_trace + (g_trace_launch++) * 148 * 16 : nullptr;
#endif
    const int digits = act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1;
    // One persistent CTA per SM, each owning a contiguous slice of at least one row group.
    const unsigned grid = gather ? gather->grid
                                 : std::max(1u, std::min<unsigned>((total_rows + zk::kGemvWarps - 1) / zk::kGemvWarps, static_cast<unsigned>(s.sm_count) * s.ctas_per_sm));
    const size_t smem = zk::gemv_q8_0_smem_bytes(nseg, static_cast<int>(tokens), digits)
                        + (gather ? zk::gather_stash_bytes(total_rows, grid, static_cast<int>(tokens)) : 0);
    if (smem > s.smem_optin) return set_error(s, "gemv: activation rows do not fit shared memory (columns x tokens too large)");
    const cudaError_t e = digits == 2 ? dispatch_batch<2>(static_cast<int>(tokens), p, grid, smem, st, s.pdl)
                                      : dispatch_batch<1>(static_cast<int>(tokens), p, grid, smem, st, s.pdl);
    if (e != cudaSuccess) return set_error(s, std::string("gemv launch: ") + cudaGetErrorString(e));
    ++s.stats.dispatches;
    return true;
}


// ---- a list of products in one persistent launch (gemv_list.cuh) ---------------------------------------------------

template <int kDigits, int kItems>
cudaError_t launch_gemv_list(const zk::GemvListParams<kItems>& p, unsigned grid, size_t smem, cudaStream_t st, bool pdl) {
    auto* fn = &zk::gemv_q8_0_list_kernel<kDigits, kItems>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(zk::kListThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, fn, p);
}

// One launch for items [first, first + n) of the list.
template <int kItems>
cudaError_t launch_list_piece(State& s, const zen_cuda_gemv_list& list, size_t first, size_t n, cudaStream_t st) {
    static zk::GemvListParams<kItems> p;   // 30 KB for the long instantiation: not on the stack; calls are serialised by the backend mutex
    std::memcpy(p.items, list.items.data() + first, n * sizeof(zk::GemvListItem));
    p.nitems = static_cast<uint32_t>(n);
    p.kpad_blocks = list.kpad_blocks;
    p.counter = list.d_counter;
    p.error_word = s.d_error;
    p.ahead_units = s.list_ahead_units;
#ifdef ZK_TRACE
    p.trace = g_trace;
#endif
    // one CTA per SM, all resident at once: the items' dependency waits need every CTA to make progress
    const unsigned grid = static_cast<unsigned>(s.sm_count);
    return list.digits == 2 ? launch_gemv_list<2, kItems>(p, grid, list.smem, st, s.pdl) : launch_gemv_list<1, kItems>(p, grid, list.smem, st, s.pdl);
}

zen_cuda_gemv_list* list_create_locked(State& s, const zen_cuda_gemv_list_item* items, size_t count, int act_mode) {
    auto bad = [&s](const char* why) { set_error(s, std::string("gemv_list_create: ") + why); return static_cast<zen_cuda_gemv_list*>(nullptr); };
    if (!items || !count || count > 4096) return bad("bad item list");
    if (act_mode != ZEN_CUDA_ACT_INT8 && act_mode != ZEN_CUDA_ACT_FP32) return bad("bad activation mode");
    std::vector<zk::GemvListItem> host(count);
    uint32_t kpad = 0;
    uint64_t bytes = 0;
    for (size_t i = 0; i < count; ++i) {
        const zen_cuda_gemv_list_item& in = items[i];
        zk::GemvListItem& it = host[i];
        if (!in.w || !in.d_y || !in.count || in.count > zk::kMaxTasks || !in.d_x) return bad("an item needs tensors, outputs and an input");
        if (in.fusion.gate && in.fusion.norm_weight) return bad("a fused input is either SwiGLU or RMSNorm");
        if (in.fusion.swiglu_pair) return bad("a SwiGLU pair is not a list item");
        uint32_t total_rows = 0;
        for (size_t k = 0; k < in.count; ++k) {
            const zen_cuda_weights* w = in.w[k];
            if (!w || !in.d_y[k] || w->format != ZEN_CUDA_Q8_0 || w->cols != in.w[0]->cols) return bad("the tensors of an item must be Q8_0 and share their columns");
            it.task[k].codes = static_cast<const uint8_t*>(w->plane[0]);
            it.task[k].scales = static_cast<const __half*>(w->plane[1]);
            it.task[k].y = in.d_y[k];
            it.task[k].rows = static_cast<uint32_t>(w->rows);
            it.task[k].first_row = total_rows;
            total_rows += static_cast<uint32_t>(w->rows);
            bytes += w->raw_bytes + w->rows * sizeof(float);
        }
        const size_t cols = in.w[0]->cols;
        const uint32_t nb = static_cast<uint32_t>(cols / 32);
        if (in.w[0]->nb != nb || in.w[0]->nbp != ((nb + 7) & ~7u)) return bad("resident tensor has an unexpected scale pitch");
        if ((reinterpret_cast<uintptr_t>(in.d_x) | reinterpret_cast<uintptr_t>(in.fusion.gate) | reinterpret_cast<uintptr_t>(in.fusion.norm_weight)) % 16)
            return bad("inputs must be 16-byte aligned");
        bytes += cols * sizeof(float);
        it.x = in.d_x;
        it.x_gate = in.fusion.gate;
        it.norm_weight = in.fusion.norm_weight;
        it.norm_eps = in.fusion.norm_eps;
        it.flags = (in.fusion.gate ? zk::kGemvFlagSwiglu : 0u) | (in.fusion.norm_weight ? zk::kGemvFlagNorm : 0u) |
                   (in.fusion.accumulate ? zk::kGemvFlagAccumulate : 0u) | (in.depends_on_earlier_items ? zk::kListFlagDepends : 0u);
        it.K = static_cast<uint32_t>(cols);
        it.total_rows = total_rows;
        // the device does no division: the geometry of the rows in the ring and the CTAs' row cut are settled here
        const uint32_t grid = static_cast<uint32_t>(s.sm_count);
        it.rows_q = total_rows / grid;
        it.rows_rem = total_rows % grid;
        it.nb = nb;
        it.nbp = (nb + 7) & ~7u;
        it.nseg = (nb + zk::kGemvSegBlocks - 1) / zk::kGemvSegBlocks;
        it.segb = ((nb + it.nseg - 1) / it.nseg + 7) & ~7u;
        if (it.nseg == 1 && it.nb == it.nbp) it.flags |= zk::kListFlagContiguous;
        kpad = std::max(kpad, it.nseg * zk::kGemvSegBlocks);
    }
    const int digits = act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1;
    const size_t smem = zk::gemv_list_smem_bytes(kpad, digits);
    if (smem > s.smem_optin) return bad("the widest input does not fit shared memory beside the weight ring");
    auto* list = new zen_cuda_gemv_list;
    void* dev = nullptr;
    if (cudaMalloc(&dev, 16) != cudaSuccess || cudaMemset(dev, 0, 16) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        if (dev) cudaFree(dev);
        delete list;
        return bad("out of device memory");
    }
    list->d_counter = static_cast<unsigned int*>(dev);
    list->items = std::move(host);
    list->kpad_blocks = kpad;
    list->digits = digits;
    list->smem = smem;
    list->algorithmic_bytes = bytes;
    return list;
}

// ---- prefill GEMM (tcgen05) -----------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_map_2d(State& s, CUtensorMap* map, CUtensorMapDataType type, size_t elem_bytes, const void* base, uint64_t inner, uint64_t outer,
                 uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    if (!s.encode_tiled) return set_error(s, "gemm: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    const CUresult r = reinterpret_cast<EncodeTiledFn>(s.encode_tiled)(map, type, 2, const_cast<void*>(base), dims, strides, box, estr,
                                                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(s, "gemm: cuTensorMapEncodeTiled failed (" + std::to_string(static_cast<int>(r)) + ")");
    return true;
}

// Workspace of one prefill product: codes [tokens][cols] int8 (padded to 256 bytes), block-major scales [cols/32][t_ld]
// fp32 and, with two activation digits, the fine digits [tokens][cols] behind them on the next 256-byte boundary.
// Q8_0 tensors whose rows span several K segments (more than 4096 columns) and whose columns are a multiple of 256: the
// two tiled views through which the decode kernel fetches a segment of a whole row group with one copy per plane.
// Other tensors keep none (their rows are contiguous per group, or go row by row).
bool make_tile_maps(State& s, zen_cuda_weights* w) {
    if (w->cols <= static_cast<size_t>(zk::kGemvSegBlocks) * 32 || w->cols % 256 || !s.encode_tiled) return true;
    zk::GemvTileMaps maps;
    std::memset(&maps, 0, sizeof maps);
    const auto encode = reinterpret_cast<EncodeTiledFn>(s.encode_tiled);
    for (int k = 0; k < 4; ++k) {   // boxes of 8, 4, 2 and 1 rows
        const cuuint32_t box_rows = static_cast<cuuint32_t>(zk::kTeamWarps) >> k;
        {
            const cuuint64_t dims[3] = {256, w->cols / 256, w->rows};
            const cuuint64_t strides[2] = {256, w->cols};
            const cuuint32_t box[3] = {256, static_cast<cuuint32_t>(zk::kGemvSegBlocks * 32 / 256), box_rows};
            const cuuint32_t estr[3] = {1, 1, 1};
            const CUresult r = encode(&maps.codes[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w->plane[0], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return true;   // no maps: the rows go one copy each, as before
        }
        {
            const cuuint64_t dims[2] = {w->nbp, w->rows};
            const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w->nbp) * 2};
            const cuuint32_t box[2] = {static_cast<cuuint32_t>(zk::kGemvSegBlocks), box_rows};
            const cuuint32_t estr[2] = {1, 1};
            const CUresult r = encode(&maps.scales[k], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->plane[1], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return true;
        }
    }
    ZC_CUDA(s, cudaMalloc(&w->d_tile_maps, sizeof maps));
    ZC_CUDA(s, cudaMemcpy(w->d_tile_maps, &maps, sizeof maps, cudaMemcpyHostToDevice));
    w->device_bytes += sizeof maps;
    return true;
}

// The same for the planes of the Q4_0 / Q6_K / Q4_K / Q5_K kernel (zk::KqTileMaps): per plane the row pitch and the bytes
// of one 4096-column segment; planes wider than 256 bytes a segment need a pitch that is a multiple of 256.
bool make_kq_tile_maps(State& s, zen_cuda_weights* w) {
    if (w->cols <= static_cast<size_t>(zk::kKqSegElems) || !s.encode_tiled) return true;
    const int kf = w->kernel_format;
    size_t pitch[4] = {0, 0, 0, 0}, seg[4] = {0, 0, 0, 0};
    int planes = 0;
    const size_t K = w->cols, E = zk::kKqSegElems;
    if (kf == ZEN_CUDA_Q4_0) { planes = 2; pitch[0] = K / 2; seg[0] = E / 2; pitch[1] = size_t(w->nbp) * 2; seg[1] = E / 32 * 2; }
    else if (kf == ZEN_CUDA_Q6_K) { planes = 4; pitch[0] = K / 2; seg[0] = E / 2; pitch[1] = K / 4; seg[1] = E / 4; pitch[2] = K / 16; seg[2] = E / 16; pitch[3] = size_t(w->nbp) * 2; seg[3] = E / 256 * 2; }
    else if (kf == zk::kFormatQ6KCodes) { planes = 3; pitch[0] = K; seg[0] = E; pitch[1] = K / 16; seg[1] = E / 16; pitch[2] = size_t(w->nbp) * 2; seg[2] = E / 256 * 2; }
    else if (kf == ZEN_CUDA_Q4_K) { planes = 3; pitch[0] = K / 2; seg[0] = E / 2; pitch[1] = K / 16; seg[1] = E / 16; pitch[2] = size_t(w->nbp) * 4; seg[2] = E / 256 * 4; }
    else if (kf == ZEN_CUDA_Q5_K) { planes = 4; pitch[0] = K / 2; seg[0] = E / 2; pitch[1] = K / 8; seg[1] = E / 8; pitch[2] = K / 16; seg[2] = E / 16; pitch[3] = size_t(w->nbp) * 4; seg[3] = E / 256 * 4; }
    else return true;
    for (int pl = 0; pl < planes; ++pl)
        if (pitch[pl] % 16 || (seg[pl] > 256 && pitch[pl] % 256)) return true;   // no maps: the rows go one copy each
    zk::KqTileMaps maps;
    std::memset(&maps, 0, sizeof maps);
    const auto encode = reinterpret_cast<EncodeTiledFn>(s.encode_tiled);
    for (int pl = 0; pl < planes; ++pl) {
        for (int k = 0; k < 4; ++k) {
            const cuuint32_t box_rows = 8u >> k;
            CUresult r;
            if (seg[pl] <= 256) {
                const cuuint64_t dims[2] = {pitch[pl], w->rows};
                const cuuint64_t strides[1] = {pitch[pl]};
                const cuuint32_t box[2] = {static_cast<cuuint32_t>(seg[pl]), box_rows};
                const cuuint32_t estr[2] = {1, 1};
                r = encode(&maps.map[pl][k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->plane[pl], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            } else {
                const cuuint64_t dims[3] = {256, pitch[pl] / 256, w->rows};
                const cuuint64_t strides[2] = {256, pitch[pl]};
                const cuuint32_t box[3] = {256, static_cast<cuuint32_t>(seg[pl] / 256), box_rows};
                const cuuint32_t estr[3] = {1, 1, 1};
                r = encode(&maps.map[pl][k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w->plane[pl], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            }
            if (r != CUDA_SUCCESS) return true;   // no maps: the rows go one copy each
        }
    }
    ZC_CUDA(s, cudaMalloc(&w->d_tile_maps, sizeof maps));
    ZC_CUDA(s, cudaMemcpy(w->d_tile_maps, &maps, sizeof maps, cudaMemcpyHostToDevice));
    w->device_bytes += sizeof maps;
    return true;
}

size_t gemm_ws_bytes(size_t tokens, size_t cols, int digits = 1) {
    const size_t t_ld = (tokens + 3) & ~size_t(3);
    const size_t codes = (tokens * cols + 255) & ~size_t(255);
    const size_t one = codes + (cols / 32) * t_ld * sizeof(float);
    return digits == 2 ? ((one + 255) & ~size_t(255)) + codes : one;
}

// The shared-memory opt-in of the GEMM kernel; done once, at start-up (it loads the kernel's module, which may allocate).
template <int kNTile, int kDigits = 1, bool kQ6K = false, bool kOffsets = false>
cudaError_t configure_gemm() {
    static bool configured = false;
    if (configured) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(&zk::gemm_q8_0_i8_kernel<kNTile, kDigits, kQ6K, kOffsets>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(zk::gemm_smem_bytes(kNTile, kDigits, kOffsets)));
    if (e == cudaSuccess) configured = true;
    return e;
}

template <int kNTile, int kDigits = 1, bool kQ6K = false, bool kOffsets = false>
cudaError_t launch_gemm(const zk::GemmParams& p, unsigned grid, cudaStream_t st) {
    const cudaError_t e = configure_gemm<kNTile, kDigits, kQ6K, kOffsets>();
    if (e != cudaSuccess) return e;
    zk::gemm_q8_0_i8_kernel<kNTile, kDigits, kQ6K, kOffsets><<<grid, zk::kGemmThreads, zk::gemm_smem_bytes(kNTile, kDigits, kOffsets), st>>>(p);
    return cudaGetLastError();
}

// ---- the group-scale kernel (gemm_groups.cuh) ---------------------------------------------------------------------------
// Workspace: xh | xl ([tokens][cols] int8 each, padded to 256 bytes) | activation units [cols / 256][t_ld] fp32, t_ld =
// tokens rounded up to whole 128-column tiles.
size_t gemm_groups_ws_bytes(size_t tokens, size_t cols) {
    const size_t t_ld = (tokens + zk::kGgNTile - 1) / zk::kGgNTile * zk::kGgNTile;
    return 2 * ((tokens * cols + 255) & ~size_t(255)) + (cols / zk::kGgGroup) * t_ld * sizeof(float);
}

// Makes sure the tensor's two-digit planes exist.  They are built once, on `st`, and the call returns after the build has
// run (other streams may use them at once).  False without an error: not now (the stream is being captured, or memory is
// short) -- the caller takes the per-block kernel.
bool ensure_group_digits(State& s, const zen_cuda_weights* w, cudaStream_t st) {
    if (w->g_hi) return true;
    const int kf = w->kernel_format;
    if (w->cols % zk::kGgGroup || kf == ZEN_CUDA_Q6_K) return false;      // Q6_K with the file's planes: no builder
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return false;
    const size_t n = w->rows * w->cols, groups = w->cols / zk::kGgGroup;
    if (s.vram_budget && s.stats.weight_bytes + 2 * n > s.vram_budget) return false;   // the planes count as residency; no eviction for them
    void *hi = nullptr, *lo = nullptr;
    float* unit = nullptr;
    if (cudaMalloc(&hi, n) != cudaSuccess || cudaMalloc(&lo, n) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&unit), w->rows * groups * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        if (hi) cudaFree(hi);
        if (lo) cudaFree(lo);
        if (unit) cudaFree(unit);
        return false;
    }
    const size_t warps = w->rows * groups;
    const unsigned dgrid = static_cast<unsigned>((warps + 7) / 8);
    const uint32_t K = static_cast<uint32_t>(w->cols);
    const auto pl = [&](int i) { return static_cast<const uint8_t*>(w->plane[i]); };
    int8_t* h8 = static_cast<int8_t*>(hi);
    int8_t* l8 = static_cast<int8_t*>(lo);
    if (kf == ZEN_CUDA_Q8_0)
        zk::group_digits_q8_0_kernel<<<dgrid, 256, 0, st>>>(static_cast<const int8_t*>(w->plane[0]), static_cast<const __half*>(w->plane[1]), w->nbp, h8, l8, unit,
                                                            w->rows, K);
    else if (kf == ZEN_CUDA_Q4_0)
        zk::group_digits_kq_kernel<2><<<dgrid, 256, 0, st>>>(pl(0), pl(1), nullptr, nullptr, w->nbp, h8, l8, unit, w->rows, K);
    else if (kf == zk::kFormatQ6KCodes)
        zk::group_digits_kq_kernel<114><<<dgrid, 256, 0, st>>>(pl(0), pl(1), pl(2), nullptr, w->nbp, h8, l8, unit, w->rows, K);
    else if (kf == ZEN_CUDA_Q4_K)
        zk::group_digits_kq_kernel<12><<<dgrid, 256, 0, st>>>(pl(0), pl(1), pl(2), nullptr, w->nbp, h8, l8, unit, w->rows, K);
    else
        zk::group_digits_kq_kernel<13><<<dgrid, 256, 0, st>>>(pl(0), pl(1), pl(2), pl(3), w->nbp, h8, l8, unit, w->rows, K);
    const bool ok = cudaGetLastError() == cudaSuccess && cudaStreamSynchronize(st) == cudaSuccess;
    ++s.stats.dispatches;
    if (!ok) { cudaFree(hi); cudaFree(lo); cudaFree(unit); return false; }
    w->g_hi = hi; w->g_lo = lo; w->g_unit = unit;
    w->g_bytes = 2 * n + w->rows * groups * sizeof(float);
    s.stats.weight_bytes += w->g_bytes;
    return true;
}

cudaError_t configure_gemm_groups() {
    static bool configured = false;
    if (configured) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(&zk::gemm_groups_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(zk::gemm_groups_smem_bytes()));
    if (e == cudaSuccess) configured = true;
    return e;
}

// All tensors have their two-digit planes (ensure_group_digits) and share the columns; `ws` holds gemm_groups_ws_bytes.
bool enqueue_gemm_groups(State& s, const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x, size_t tokens, uint8_t* ws,
                         cudaStream_t st, int act_mode) {
    const size_t cols = w[0]->cols;
    const uint32_t groups = static_cast<uint32_t>(cols / zk::kGgGroup);
    const uint32_t n_tiles = static_cast<uint32_t>((tokens + zk::kGgNTile - 1) / zk::kGgNTile), t_ld = n_tiles * zk::kGgNTile;
    const size_t plane = (tokens * cols + 255) & ~size_t(255);
    int8_t* xh = reinterpret_cast<int8_t*>(ws);
    int8_t* xl = reinterpret_cast<int8_t*>(ws + plane);
    float* x_unit = reinterpret_cast<float*>(ws + 2 * plane);
    if (tokens % zk::kGgNTile)      // the columns past the last token carry a zero unit
        if (cudaMemsetAsync(x_unit, 0, static_cast<size_t>(groups) * t_ld * sizeof(float), st) != cudaSuccess) return set_error(s, "gemm: clearing the activation units failed");
    const size_t warps = tokens * groups;
    zk::group_digits_acts_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, st>>>(d_x, xh, xl, x_unit, static_cast<uint32_t>(tokens), static_cast<uint32_t>(cols),
                                                                                        t_ld, act_mode == ZEN_CUDA_ACT_INT8 ? 1 : 0);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm: activation digits launch failed");
    ++s.stats.dispatches;
    if (configure_gemm_groups() != cudaSuccess) return set_error(s, "gemm: shared-memory opt-in failed");
    for (size_t i0 = 0; i0 < count; i0 += zk::kGemmMaxTensors) {
        const size_t n = std::min<size_t>(zk::kGemmMaxTensors, count - i0);
        zk::GroupGemmParams p{};
        uint32_t m_tiles = 0;
        for (size_t j = 0; j < static_cast<size_t>(zk::kGemmMaxTensors); ++j) {
            if (j >= n) { p.m_start[j] = 0xffffffffu; continue; }
            const zen_cuda_weights* wt = w[i0 + j];
            if (!make_map_2d(s, &p.map_wh[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wt->g_hi, cols, wt->rows, cols, zk::kGemmKTile, zk::kGemmM, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
            if (!make_map_2d(s, &p.map_wl[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wt->g_lo, cols, wt->rows, cols, zk::kGemmKTile, zk::kGemmM, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
            p.w_unit[j] = wt->g_unit;
            p.out[j] = d_out[i0 + j];
            p.rows[j] = static_cast<uint32_t>(wt->rows);
            p.m_start[j] = m_tiles;
            m_tiles += (p.rows[j] + zk::kGemmM - 1) / zk::kGemmM;
        }
        if (!make_map_2d(s, &p.map_xh, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xh, cols, tokens, cols, zk::kGemmKTile, zk::kGgNTile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        if (!make_map_2d(s, &p.map_xl, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xl, cols, tokens, cols, zk::kGemmKTile, zk::kGgNTile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        p.x_unit = x_unit;
        p.tensors = static_cast<uint32_t>(n);
        p.tokens = static_cast<uint32_t>(tokens);
        p.groups = groups;
        p.t_ld = t_ld;
        p.m_tiles = m_tiles;
        p.n_tiles = n_tiles;
        p.error_word = s.d_error;
        const unsigned tiles = p.m_tiles * p.n_tiles;
        const unsigned grid = std::min<unsigned>(tiles, static_cast<unsigned>(s.sm_count));
        p.stream_k = (s.gemm_stream_k && tiles % grid != 0 && static_cast<uint64_t>(tiles) * groups / grid >= groups) ? 1u : 0u;
        if (p.stream_k) {
            zk::gg_zero_split_tiles_kernel<<<grid, 256, 0, st>>>(p);
            ++s.stats.dispatches;
        }
        zk::gemm_groups_kernel<<<grid, zk::kGgThreads, zk::gemm_groups_smem_bytes(), st>>>(p);
        if (cudaGetLastError() != cudaSuccess) return set_error(s, std::string("gemm launch: ") + cudaGetErrorString(cudaGetLastError()));
        ++s.stats.dispatches;
    }
    return true;
}

// One tensor of any format through the group-scale kernel when it can be: whole 256-weight groups, room in the workspace,
// the tensor's two-digit planes at hand or buildable now.  `launched` tells the caller whether it still has to take its own path.
bool try_gemm_groups(State& s, const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, uint8_t* ws, size_t ws_bytes, cudaStream_t st,
                     bool& launched) {
    launched = false;
    if (!s.gemm_groups || !w || w->cols % zk::kGgGroup || ws_bytes < gemm_groups_ws_bytes(tokens, w->cols) || !ensure_group_digits(s, w, st)) return true;
    launched = true;
    const zen_cuda_weights* wp[1] = {w};
    float* outs[1] = {d_out};
    return enqueue_gemm_groups(s, wp, outs, 1, d_x, tokens, ws, st, ZEN_CUDA_ACT_FP32);
}

// What a caller's workspace must hold for either kernel.
size_t gemm_ws_bytes_any(const State& s, size_t tokens, size_t cols, int act_mode) {
    const size_t per_block = gemm_ws_bytes(tokens, cols, act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1);
    return s.gemm_groups && cols % zk::kGgGroup == 0 ? std::max(per_block, gemm_groups_ws_bytes(tokens, cols)) : per_block;
}

// Quantises d_x [tokens][cols] into the workspace `ws` (gemm_ws_bytes) and enqueues one GEMM per tensor.
// Everything is stream-ordered on `st`; `ws` must stay untouched until the work has run.  act_mode ZEN_CUDA_ACT_FP32:
// two activation digits (the workspace is the larger one, gemm_ws_bytes(..., 2)).
// ws_bytes: what `ws` holds; with room for gemm_groups_ws_bytes, whole 256-weight groups and every tensor's two-digit planes
// at hand the product goes through the group-scale kernel, otherwise through the per-block kernel below.
bool enqueue_gemm_q8_0(State& s, const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x, size_t tokens,
                       uint8_t* ws, cudaStream_t st, int act_mode = ZEN_CUDA_ACT_INT8, size_t ws_bytes = 0) {
    if (!count || !tokens || !d_x || !ws) return set_error(s, "gemm: bad arguments");
    if (act_mode != ZEN_CUDA_ACT_INT8 && act_mode != ZEN_CUDA_ACT_FP32) return set_error(s, "gemm: bad activation mode");
    if (s.gemm_groups && w[0] && w[0]->cols % zk::kGgGroup == 0 && ws_bytes >= gemm_groups_ws_bytes(tokens, w[0]->cols)) {
        bool all = true;
        for (size_t i = 0; i < count && all; ++i)
            all = w[i] && d_out[i] && w[i]->format == ZEN_CUDA_Q8_0 && w[i]->cols == w[0]->cols && ensure_group_digits(s, w[i], st);
        if (all) return enqueue_gemm_groups(s, w, d_out, count, d_x, tokens, ws, st, act_mode);
    }
    const int digits = act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1;
    const size_t cols = w[0]->cols;
    const uint32_t nb = w[0]->nb;
    const size_t t_ld = (tokens + 3) & ~size_t(3);
    int8_t* xq = reinterpret_cast<int8_t*>(ws);
    float* xs_t = reinterpret_cast<float*>(ws + ((tokens * cols + 255) & ~size_t(255)));
    int8_t* xq2 = digits == 2 ? reinterpret_cast<int8_t*>(ws + ((gemm_ws_bytes(tokens, cols, 1) + 255) & ~size_t(255))) : nullptr;
    const size_t nblk = tokens * nb;
    zk::quantize_acts_gemm_kernel<<<static_cast<unsigned>((nblk + 7) / 8), 256, 0, st>>>(d_x, xq, xs_t, static_cast<uint32_t>(tokens), nb,
                                                                                      static_cast<uint32_t>(t_ld), xq2);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm: quantise launch failed");
    ++s.stats.dispatches;
    const uint32_t n_tile = 128u;  // tokens per tile: sixteen epilogue warps take 32 token columns each
    for (size_t i = 0; i < count; ++i)
        if (!w[i] || !d_out[i] || w[i]->format != ZEN_CUDA_Q8_0 || w[i]->cols != cols || w[i]->nbp != w[0]->nbp)
            return set_error(s, "gemm: tasks must be Q8_0 and share columns");
    // Up to kGemmMaxTensors tensors per launch: their row tiles are numbered through, so that q|k|v or gate|up fill the
    // SMs together (a 1024-row tensor alone is 32 tiles for 148 SMs).
    for (size_t i0 = 0; i0 < count; i0 += zk::kGemmMaxTensors) {
        const size_t n = std::min<size_t>(zk::kGemmMaxTensors, count - i0);
        zk::GemmParams p{};
        uint32_t m_tiles = 0;
        for (size_t j = 0; j < static_cast<size_t>(zk::kGemmMaxTensors); ++j) {
            if (j >= n) { p.m_start[j] = 0xffffffffu; continue; }
            const zen_cuda_weights* wt = w[i0 + j];
            if (!make_map_2d(s, &p.map_w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wt->plane[0], cols, wt->rows, cols, zk::kGemmKTile, zk::kGemmM,
                             CU_TENSOR_MAP_SWIZZLE_128B)) return false;
            p.w_scales[j] = static_cast<const __half*>(wt->plane[1]);
            p.out[j] = d_out[i0 + j];
            p.rows[j] = static_cast<uint32_t>(wt->rows);
            p.m_start[j] = m_tiles;
            m_tiles += (p.rows[j] + zk::kGemmM - 1) / zk::kGemmM;
        }
        if (!make_map_2d(s, &p.map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, cols, tokens, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        if (xq2 && !make_map_2d(s, &p.map_x2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq2, cols, tokens, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        if (!make_map_2d(s, &p.map_xs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, xs_t, t_ld, nb, t_ld * sizeof(float), n_tile, zk::kGemmBlocksPerTile,
                         CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
        p.tensors = static_cast<uint32_t>(n);
        p.tokens = static_cast<uint32_t>(tokens);
        p.nb = nb;
        p.nbp = w[0]->nbp;
        p.n_tile = n_tile;
        p.m_tiles = m_tiles;
        p.n_tiles = (p.tokens + n_tile - 1) / n_tile;
        p.error_word = s.d_error;
        const unsigned tiles = p.m_tiles * p.n_tiles, ktiles = (nb + zk::kGemmBlocksPerTile - 1) / zk::kGemmBlocksPerTile;
        const unsigned grid = std::min<unsigned>(tiles, static_cast<unsigned>(s.sm_count));
        // Uneven tile counts: share the K tiles evenly instead (every CTA's range must span at least one tile's worth,
        // so that no tile is cut more than once).
        p.stream_k = (s.gemm_stream_k && tiles % grid != 0 && static_cast<uint64_t>(tiles) * ktiles / grid >= ktiles) ? 1u : 0u;
        if (p.stream_k) {
            zk::gemm_zero_split_tiles_kernel<<<grid, 256, 0, st>>>(p, ktiles);
            ++s.stats.dispatches;
        }
        const cudaError_t e = digits == 2 ? launch_gemm<128, 2>(p, grid, st) : launch_gemm<128, 1>(p, grid, st);
        if (e != cudaSuccess) return set_error(s, std::string("gemm launch: ") + cudaGetErrorString(e));
        ++s.stats.dispatches;
    }
    return true;
}

// Q6_K (codes unpacked on upload) times `tokens` >= 2 activation rows on the tensor cores: every token enters as two
// columns, one per parity of the 16-weight groups (gemm_q8_0_i8.cuh), in tiles of 32 columns = 16 tokens.  The workspace
// is gemm_ws_bytes(2 * tokens, cols, 2).  Stream-ordered on `st`.
// Narrow tiles (32 columns = 16 tokens) up to kQ6kNarrowMaxTokens rows, the prefill GEMM's 128 columns (64 tokens) beyond.
constexpr size_t kQ6kNarrowMaxTokens = 16;
// From this many activation rows on the host-pointer call takes the tensor-core product: the narrow-tile kernel takes the
// same ~270 us for the 128256 x 4096 lm_head whatever the row count, the decode kernel 43 + 41 us per row.
constexpr size_t kQ6kTensorMinTokens = 7;
size_t gemm_q6k_ws_bytes(size_t tokens, size_t cols) { return std::max(gemm_ws_bytes(2 * tokens, cols, 2), gemm_groups_ws_bytes(tokens, cols)); }

bool enqueue_gemm_q6k(State& s, const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, uint8_t* ws, cudaStream_t st, size_t ws_bytes = 0) {
    if (!w || !d_out || !d_x || !ws || !tokens) return set_error(s, "gemm q6_k: bad arguments");
    {                                       // the group-scale kernel when it can be
        bool launched = false;
        if (!try_gemm_groups(s, w, d_out, d_x, tokens, ws, ws_bytes, st, launched)) return false;
        if (launched) return true;
    }
    if (w->kernel_format != zk::kFormatQ6KCodes || w->cols % 256) return set_error(s, "gemm q6_k: the tensor is not resident with its codes unpacked");
    const size_t cols = w->cols, columns = 2 * tokens;
    const uint32_t nb = static_cast<uint32_t>(cols / 32);
    const size_t t_ld = (columns + 3) & ~size_t(3);
    int8_t* xq = reinterpret_cast<int8_t*>(ws);
    float* xs_t = reinterpret_cast<float*>(ws + ((columns * cols + 255) & ~size_t(255)));
    int8_t* xq2 = reinterpret_cast<int8_t*>(ws + ((gemm_ws_bytes(columns, cols, 1) + 255) & ~size_t(255)));
    const size_t nblk = tokens * nb;
    zk::quantize_acts_q6k_gemm_kernel<<<static_cast<unsigned>((nblk + 7) / 8), 256, 0, st>>>(d_x, xq, xs_t, static_cast<uint32_t>(tokens), nb,
                                                                                          static_cast<uint32_t>(t_ld), xq2);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm q6_k: quantise launch failed");
    ++s.stats.dispatches;
    zk::GemmParams p{};
    p.m_start[0] = 0; p.m_start[1] = p.m_start[2] = 0xffffffffu;
    if (!make_map_2d(s, &p.map_w[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->plane[0], cols, w->rows, cols, zk::kGemmKTile, zk::kGemmM, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    const uint32_t n_tile = tokens <= kQ6kNarrowMaxTokens ? 32u : 128u;   // columns per tile: two per token
    if (!make_map_2d(s, &p.map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, cols, columns, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(s, &p.map_x2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq2, cols, columns, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(s, &p.map_xs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, xs_t, t_ld, nb, t_ld * sizeof(float), n_tile, zk::kGemmBlocksPerTile,
                     CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    p.w_group_scales[0] = static_cast<const int8_t*>(w->plane[1]);
    p.group_pitch = static_cast<uint32_t>(cols / 16);
    p.w_scales[0] = static_cast<const __half*>(w->plane[2]);
    p.out[0] = d_out;
    p.rows[0] = static_cast<uint32_t>(w->rows);
    p.tensors = 1;
    p.tokens = static_cast<uint32_t>(tokens);
    p.nb = nb;
    p.nbp = w->nbp;
    p.n_tile = n_tile / 2;   // tokens per tile
    p.m_tiles = (p.rows[0] + zk::kGemmM - 1) / zk::kGemmM;
    p.n_tiles = (p.tokens + p.n_tile - 1) / p.n_tile;
    p.error_word = s.d_error;
    const unsigned tiles = p.m_tiles * p.n_tiles, ktiles = nb / zk::kGemmBlocksPerTile;
    const unsigned grid = std::min<unsigned>(tiles, static_cast<unsigned>(s.sm_count));
    p.stream_k = (s.gemm_stream_k && tiles % grid != 0 && static_cast<uint64_t>(tiles) * ktiles / grid >= ktiles) ? 1u : 0u;
    if (p.stream_k) {
        zk::gemm_zero_split_tiles_kernel<<<grid, 256, 0, st>>>(p, ktiles);
        ++s.stats.dispatches;
    }
    const cudaError_t e = n_tile == 32 ? launch_gemm<32, 2, true>(p, grid, st) : launch_gemm<128, 2, true>(p, grid, st);
    if (e != cudaSuccess) return set_error(s, std::string("gemm q6_k launch: ") + cudaGetErrorString(e));
    ++s.stats.dispatches;
    return true;
}

// Q4_0 times many activation rows: the nibbles are widened to int8 codes n - 8 in scratch memory (with the tensor's own
// f16 block scales that is a Q8_0 tensor), then the Q8_0 GEMM with two activation digits, the fp32-activation arithmetic
// the reference uses for this format (generic route, src/quant.cpp:1135-1162).  The workspace holds the codes
// (rows x cols bytes, padded to 256) followed by the GEMM's own workspace.
constexpr size_t kQ4TensorMinTokens = 9;    // 14336 x 4096: 37 us up to 128 rows through the group-scale kernel (96 us with nibbles widened per call), 75 us per chunk of eight through the decode kernel
size_t gemm_q4_0_ws_bytes(size_t tokens, size_t rows, size_t cols) {
    return std::max(((rows * cols + 255) & ~size_t(255)) + gemm_ws_bytes(tokens, cols, 2), gemm_groups_ws_bytes(tokens, cols));
}

bool enqueue_gemm_q4_0(State& s, const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, uint8_t* ws, cudaStream_t st, size_t ws_bytes = 0) {
    if (!w || !d_out || !d_x || !ws || !tokens) return set_error(s, "gemm q4_0: bad arguments");
    if (w->format != ZEN_CUDA_Q4_0) return set_error(s, "gemm q4_0: not a Q4_0 tensor");
    {
        bool launched = false;
        if (!try_gemm_groups(s, w, d_out, d_x, tokens, ws, ws_bytes, st, launched)) return false;
        if (launched) return true;
    }
    const size_t blocks = w->rows * w->nb;
    zk::unpack_q4_0_codes_kernel<<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(w->plane[0]),
                                                                                             reinterpret_cast<int8_t*>(ws), blocks);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm q4_0: unpack launch failed");
    ++s.stats.dispatches;
    zen_cuda_weights as_q8 = *w;          // a view: the widened codes and the tensor's own scale plane
    as_q8.format = as_q8.kernel_format = ZEN_CUDA_Q8_0;
    as_q8.plane[0] = ws;
    as_q8.d_tile_maps = nullptr;
    const zen_cuda_weights* wp[1] = {&as_q8};
    float* outs[1] = {d_out};
    return enqueue_gemm_q8_0(s, wp, outs, 1, d_x, tokens, ws + ((w->rows * w->cols + 255) & ~size_t(255)), st, ZEN_CUDA_ACT_FP32);
}

// Q4_K / Q5_K times many activation rows: codes widened to int8 in scratch memory together with the fp32 scale and offset
// of every 32-weight sub-block (w = scale * q - offset), then the tensor-core GEMM with two activation digits whose
// epilogue also subtracts offset x (activation sum of the block).  Workspace: codes | scales | offsets | GEMM workspace |
// block-major activation sums.
constexpr size_t kK45TensorMinTokens = 9;
size_t align256(size_t n) { return (n + 255) & ~size_t(255); }
size_t gemm_k45_ws_bytes(size_t tokens, size_t rows, size_t cols) {
    const size_t t_ld = (tokens + 3) & ~size_t(3);
    return std::max(align256(rows * cols) + 2 * align256(rows * (cols / 32) * sizeof(float)) + align256(gemm_ws_bytes(tokens, cols, 2)) + (cols / 32) * t_ld * sizeof(float),
                    gemm_groups_ws_bytes(tokens, cols));
}

bool enqueue_gemm_k45(State& s, const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, uint8_t* ws, cudaStream_t st, size_t ws_bytes = 0) {
    if (!w || !d_out || !d_x || !ws || !tokens) return set_error(s, "gemm k-quant: bad arguments");
    const bool q5 = w->format == ZEN_CUDA_Q5_K;
    if (!q5 && w->format != ZEN_CUDA_Q4_K) return set_error(s, "gemm k-quant: not a Q4_K or Q5_K tensor");
    {
        bool launched = false;
        if (!try_gemm_groups(s, w, d_out, d_x, tokens, ws, ws_bytes, st, launched)) return false;
        if (launched) return true;
    }
    const size_t rows = w->rows, cols = w->cols;
    const uint32_t nsb = w->nb, nb = static_cast<uint32_t>(cols / 32);
    int8_t* codes = reinterpret_cast<int8_t*>(ws);
    float* scales = reinterpret_cast<float*>(ws + align256(rows * cols));
    float* offsets = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scales) + align256(rows * nb * sizeof(float)));
    uint8_t* gws = reinterpret_cast<uint8_t*>(offsets) + align256(rows * nb * sizeof(float));
    float* zs_t = reinterpret_cast<float*>(gws + align256(gemm_ws_bytes(tokens, cols, 2)));
    const size_t threads = rows * nsb * 4;
    const unsigned ugrid = static_cast<unsigned>((threads + 255) / 256);
    if (q5)
        zk::unpack_k45_codes_kernel<true><<<ugrid, 256, 0, st>>>(static_cast<const uint8_t*>(w->plane[0]), static_cast<const uint8_t*>(w->plane[1]),
                                                                 static_cast<const uint8_t*>(w->plane[2]), static_cast<const uint32_t*>(w->plane[3]), codes,
                                                                 scales, offsets, rows, nsb, w->nbp);
    else
        zk::unpack_k45_codes_kernel<false><<<ugrid, 256, 0, st>>>(static_cast<const uint8_t*>(w->plane[0]), nullptr, static_cast<const uint8_t*>(w->plane[1]),
                                                                  static_cast<const uint32_t*>(w->plane[2]), codes, scales, offsets, rows, nsb, w->nbp);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm k-quant: unpack launch failed");
    ++s.stats.dispatches;
    const size_t t_ld = (tokens + 3) & ~size_t(3);
    int8_t* xq = reinterpret_cast<int8_t*>(gws);
    float* xs_t = reinterpret_cast<float*>(gws + ((tokens * cols + 255) & ~size_t(255)));
    int8_t* xq2 = reinterpret_cast<int8_t*>(gws + ((gemm_ws_bytes(tokens, cols, 1) + 255) & ~size_t(255)));
    const size_t nblk = tokens * nb;
    zk::quantize_acts_gemm_kernel<<<static_cast<unsigned>((nblk + 7) / 8), 256, 0, st>>>(d_x, xq, xs_t, static_cast<uint32_t>(tokens), nb,
                                                                                      static_cast<uint32_t>(t_ld), xq2, zs_t);
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "gemm k-quant: quantise launch failed");
    ++s.stats.dispatches;
    const uint32_t n_tile = 128u;
    zk::GemmParams p{};
    p.m_start[0] = 0; p.m_start[1] = p.m_start[2] = 0xffffffffu;
    if (!make_map_2d(s, &p.map_w[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, cols, rows, cols, zk::kGemmKTile, zk::kGemmM, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(s, &p.map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, cols, tokens, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(s, &p.map_x2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq2, cols, tokens, cols, zk::kGemmKTile, n_tile, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(s, &p.map_xs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, xs_t, t_ld, nb, t_ld * sizeof(float), n_tile, zk::kGemmBlocksPerTile, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    if (!make_map_2d(s, &p.map_zs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, zs_t, t_ld, nb, t_ld * sizeof(float), n_tile, zk::kGemmBlocksPerTile, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    p.w_scales32[0] = scales;
    p.w_offsets[0] = offsets;
    p.out[0] = d_out;
    p.rows[0] = static_cast<uint32_t>(rows);
    p.tensors = 1;
    p.tokens = static_cast<uint32_t>(tokens);
    p.nb = nb;
    p.nbp = nb;
    p.n_tile = n_tile;
    p.m_tiles = (p.rows[0] + zk::kGemmM - 1) / zk::kGemmM;
    p.n_tiles = (p.tokens + n_tile - 1) / n_tile;
    p.error_word = s.d_error;
    const unsigned tiles = p.m_tiles * p.n_tiles, ktiles = nb / zk::kGemmBlocksPerTile;
    const unsigned grid = std::min<unsigned>(tiles, static_cast<unsigned>(s.sm_count));
    p.stream_k = (s.gemm_stream_k && tiles % grid != 0 && static_cast<uint64_t>(tiles) * ktiles / grid >= ktiles) ? 1u : 0u;
    if (p.stream_k) {
        zk::gemm_zero_split_tiles_kernel<<<grid, 256, 0, st>>>(p, ktiles);
        ++s.stats.dispatches;
    }
    const cudaError_t e = launch_gemm<128, 2, false, true>(p, grid, st);
    if (e != cudaSuccess) return set_error(s, std::string("gemm k-quant launch: ") + cudaGetErrorString(e));
    ++s.stats.dispatches;
    return true;
}

// Scratch of the allocation-free GEMM entry point: part of the library image, one copy per GPU that loads it.
// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[ZEN_CUDA_NOALLOC_SCRATCH_BYTES];

// Device address of g_noalloc_scratch on the current device, looked up once per device.
bool noalloc_scratch_address(State& s, uint8_t** out) {
    constexpr int kMaxDevices = 64;
    static uint8_t* by_device[kMaxDevices] = {};
    int dev = -1;
    ZC_CUDA(s, cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return set_error(s, "noalloc: unexpected device index");
    if (dev != s.device) return set_error(s, "noalloc: the calling thread's current device is not the backend's device");
    if (!by_device[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return set_error(s, std::string("noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        by_device[dev] = static_cast<uint8_t*>(p);
    }
    *out = by_device[dev];
    return true;
}

// Called once while the backend starts (allocating is still allowed there): resolves the scratch array's address on the
// backend's device, opts the GEMM kernel into its shared memory and loads the code of every kernel the entry point
// launches, so that the entry point itself never triggers a lazy module load.
bool warm_noalloc_path(State& s) {
    uint8_t* scratch = nullptr;
    if (!noalloc_scratch_address(s, &scratch)) return false;
    ZC_CUDA(s, configure_gemm<128>());
    cudaFuncAttributes attr{};
    ZC_CUDA(s, cudaFuncGetAttributes(&attr, zk::quantize_acts_gemm_kernel));
    ZC_CUDA(s, cudaFuncGetAttributes(&attr, zk::gemm_zero_split_tiles_kernel));
    return true;
}

void drop_host_graphs(State& s) {
    for (auto& kv : s.host_graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    s.host_graphs.clear();
}

bool ensure_gemm_ws(State& s, size_t bytes) {
    if (bytes <= s.d_gemm_ws_bytes) return true;
    if (s.d_gemm_ws) { cudaStreamSynchronize(s.stream); cudaFree(s.d_gemm_ws); }
    s.d_gemm_ws = nullptr; s.d_gemm_ws_bytes = 0;
    ZC_CUDA(s, cudaMalloc(reinterpret_cast<void**>(&s.d_gemm_ws), bytes));
    s.d_gemm_ws_bytes = bytes;
    return true;
}

bool ensure_scratch(State& s, size_t x_bytes, size_t y_bytes) {
    const auto t0 = clock_type::now();
    if (x_bytes > s.d_x_bytes || y_bytes > s.d_y_bytes) { cudaStreamSynchronize(s.stream); drop_host_graphs(s); }   // captured launches hold the old addresses
    if (x_bytes > s.d_x_bytes) {
        if (s.d_x) cudaFree(s.d_x);
        s.d_x = nullptr; s.d_x_bytes = 0;
        ZC_CUDA(s, cudaMalloc(reinterpret_cast<void**>(&s.d_x), x_bytes));
        s.d_x_bytes = x_bytes;
    }
    if (y_bytes > s.d_y_bytes) {
        if (s.d_y) cudaFree(s.d_y);
        s.d_y = nullptr; s.d_y_bytes = 0;
        ZC_CUDA(s, cudaMalloc(reinterpret_cast<void**>(&s.d_y), (y_bytes + 255) & ~size_t(255)));
        s.d_y_bytes = y_bytes;
    }
    const size_t need = std::max(x_bytes, y_bytes);
    if (need > s.h_stage_bytes) {
        if (s.h_stage) cudaFreeHost(s.h_stage);
        s.h_stage = nullptr; s.h_stage_bytes = 0;
        ZC_CUDA(s, cudaHostAlloc(reinterpret_cast<void**>(&s.h_stage), need, cudaHostAllocDefault));
        s.h_stage_bytes = need;
    }
    s.stats.alloc_us += us_since(t0);
    return true;
}

constexpr size_t kDirectResultBytes = size_t(1) << 20;  // results up to this size are written to host memory by the kernel itself

constexpr size_t kDirectInputBytes = size_t(256) << 10;  // activations up to this size are fetched from host memory by a kernel

// Launched with programmatic stream serialisation right behind the product: resident early, it sleeps until the
// product grid has completed, copies the result from HBM to mapped host memory in full lines (the product kernels
// write one float per row from different warps, which would cross PCIe as thousands of 4-byte writes), and then
// raises the sequence number.  One CTA.
__global__ void __launch_bounds__(1024) copy_out_publish_kernel(float4* __restrict__ host_dst, const float4* __restrict__ src, size_t n16,
                                                                volatile unsigned* done, unsigned* seq_counter) {
    zk::pdl_wait();
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) host_dst[i] = __ldcg(src + i);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {   // the number of this result: counted on the device, so that a captured launch can be replayed
        const unsigned seq = *seq_counter + 1;
        *seq_counter = seq;
        *done = seq;
    }
}

// Fetches the activations from mapped host memory into HBM.  It lets the next launch start at once: the product
// kernels stream their weights (which do not depend on the activations) while this copy crosses PCIe, and only their
// activation read waits for it (griddepcontrol.wait).
__global__ void stage_in_kernel(float4* __restrict__ dst, const float4* __restrict__ src, size_t n) {
    zk::pdl_launch_dependents();
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = src[i];
}

bool ensure_direct_result(State& s, size_t bytes) {
    if (!s.h_input) {
        ZC_CUDA(s, cudaHostAlloc(reinterpret_cast<void**>(&s.h_input), kDirectInputBytes, cudaHostAllocMapped));
        ZC_CUDA(s, cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.d_input), s.h_input, 0));
    }
    if (!s.d_seq) {
        ZC_CUDA(s, cudaMalloc(reinterpret_cast<void**>(&s.d_seq), 16));
        ZC_CUDA(s, cudaMemset(s.d_seq, 0, 16));
        ZC_CUDA(s, cudaDeviceSynchronize());
        s.done_seq = 0;
    }
    if (!s.h_done) {
        unsigned* h = nullptr;
        ZC_CUDA(s, cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped));
        *h = 0;
        s.h_done = h;
        ZC_CUDA(s, cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.d_done), h, 0));
    }
    if (bytes > s.h_result_bytes) {
        if (s.h_result) { cudaStreamSynchronize(s.stream); cudaFreeHost(s.h_result); drop_host_graphs(s); }
        s.h_result = nullptr; s.d_result = nullptr; s.h_result_bytes = 0;
        const size_t cap = (std::max(bytes, size_t(64) << 10) + 255) & ~size_t(255);   // the copy-out kernel moves whole 16-byte words
        ZC_CUDA(s, cudaHostAlloc(reinterpret_cast<void**>(&s.h_result), cap, cudaHostAllocMapped));
        ZC_CUDA(s, cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.d_result), s.h_result, 0));
        s.h_result_bytes = cap;
    }
    return true;
}

// Waits for publish_done_kernel(seq): polls the mapped word for a while, then falls back to a stream synchronise
// (which also surfaces a failed launch or a device fault as an error instead of an endless poll).
bool wait_done(State& s, unsigned seq) {
    const auto t0 = clock_type::now();
    unsigned spins = 0;
    while (*s.h_done != seq) {
        if ((++spins & 1023u) == 0 && us_since(t0) > 2000) {
            ZC_CUDA(s, cudaStreamSynchronize(s.stream));
            if (*s.h_done != seq) {   // a launch in the chain failed: take the device's count, so that later calls agree with it again
                unsigned now = 0;
                if (cudaMemcpy(&now, s.d_seq, sizeof now, cudaMemcpyDeviceToHost) == cudaSuccess) s.done_seq = now;
                return set_error(s, "result flag was not raised");
            }
            break;
        }
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#endif
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    return true;
}

// Launch with programmatic stream serialisation (the kernel calls griddepcontrol.wait before it touches memory).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(State& s, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = s.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

bool check_error_word(State& s) {
    if (*s.h_error == 0) return true;
    const int code = *s.h_error;
    *s.h_error = 0;
    return set_error(s, std::string("device-side error word: ") + zen_cuda_error_name(code) + " (code " + std::to_string(code) + ")");
}

// Resolves every tensor of one submission before anything is queued.  An eviction in the middle frees the tensors
// resolved before it, so the pass is repeated once; a submission that evicts again does not fit the budget as a whole.
// (The reference resolves first and launches after for the same reason, hip_backend.hip:625-636 and :784-797.)
bool lookup_all_locked(State& s, int fmt, const uint8_t* const* weights, const size_t* rows, size_t count, size_t cols, const zen_cuda_weights** w) {
    for (int pass = 0; pass < 2; ++pass) {
        const uint64_t before = s.evictions;
        for (size_t i = 0; i < count; ++i) {
            w[i] = lookup_locked(s, fmt, weights[i], rows[i], cols);
            if (!w[i]) return false;
        }
        if (s.evictions == before) return true;
    }
    return set_error(s, "the tensors of one submission do not fit the residency budget together");
}

// Host-pointer batched product: `count` tensors sharing `tokens` activation rows.
// Outputs are token-major [tokens][rows_i] in the caller's buffers.
bool host_product(State& s, int fmt, const float* x, const uint8_t* const* weights, float* const* ys, const size_t* rows,
                  size_t count, size_t tokens, size_t cols, int act_mode) {
    if (!x || !weights || !ys || !rows || !count || count > zk::kMaxTasks || !tokens || !cols) return set_error(s, "bad arguments");
    if (cols % block_elems(fmt)) return set_error(s, "columns are not block aligned");
    const zen_cuda_weights* w[zk::kMaxTasks];
    size_t total_rows = 0;
    for (size_t i = 0; i < count; ++i) {
        if (!weights[i] || !ys[i] || !rows[i]) return set_error(s, "bad task");
        total_rows += rows[i];
    }
    if (!lookup_all_locked(s, fmt, weights, rows, count, cols, w)) return false;
    const size_t x_bytes = tokens * cols * sizeof(float), y_bytes = tokens * total_rows * sizeof(float);
    const bool direct = y_bytes <= kDirectResultBytes;
    if (!ensure_scratch(s, x_bytes, y_bytes)) return false;
    if (direct && !ensure_direct_result(s, y_bytes)) return false;
    float* const d_result = s.d_y;
    const float* const h_result = direct ? s.h_result : s.h_stage;
    // Token chunks of up to eight rows per launch; each task's device output is [tokens][rows_i].
    float* d_out[zk::kMaxTasks];
    size_t off = 0;
    for (size_t i = 0; i < count; ++i) { d_out[i] = d_result + off; off += tokens * rows[i]; }
    const size_t chunk = max_tokens_per_launch(s, w[0]->kernel_format, cols, act_mode);
    if (!chunk) return set_error(s, "columns too large: one activation row does not fit shared memory");
    // More than one decode launch worth of int8-activation Q8_0 tokens: the tensor-core GEMM.
    // Q6_K with its codes unpacked: the tensor-core product from kQ6kTensorMinTokens activation rows on (fewer stream faster
    // through the decode kernel).
    bool q6k_tensor_path = s.use_gemm && fmt == ZEN_CUDA_Q6_K && tokens >= kQ6kTensorMinTokens;
    for (size_t i = 0; i < count; ++i) q6k_tensor_path = q6k_tensor_path && w[i]->kernel_format == zk::kFormatQ6KCodes;   // the file's planes: decode kernel
    const bool q4_tensor_path = s.use_gemm && fmt == ZEN_CUDA_Q4_0 && tokens >= kQ4TensorMinTokens && cols % 128 == 0;
    const bool k45_tensor_path = s.use_gemm && (fmt == ZEN_CUDA_Q4_K || fmt == ZEN_CUDA_Q5_K) && tokens >= kK45TensorMinTokens;
    const bool tensor_path = q6k_tensor_path || q4_tensor_path || k45_tensor_path || (s.use_gemm && fmt == ZEN_CUDA_Q8_0 && tokens > 8);   // Q8_0: either activation mode
    const bool fetch_by_kernel = direct && x_bytes <= kDirectInputBytes;

    // The three launches of a small call (fetch the activations, the product, copy the result out and publish it).
    auto enqueue_chain = [&]() -> bool {
        const size_t n16 = x_bytes / sizeof(float4);
        stage_in_kernel<<<static_cast<unsigned>(std::min<size_t>((n16 + 255) / 256, 32)), 256, 0, s.stream>>>(
            reinterpret_cast<float4*>(s.d_x), reinterpret_cast<const float4*>(s.d_input), n16);
        ++s.stats.dispatches;
        if (cudaGetLastError() != cudaSuccess) return set_error(s, "activation fetch launch failed");
        if (!enqueue_gemv(s, w, d_out, count, s.d_x, tokens, act_mode, s.stream)) return false;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(1024);
        cfg.stream = s.stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = s.pdl ? 1 : 0;
        ++s.stats.dispatches;
        if (cudaLaunchKernelEx(&cfg, copy_out_publish_kernel, reinterpret_cast<float4*>(s.d_result), reinterpret_cast<const float4*>(s.d_y),
                               (y_bytes + 15) / 16, s.d_done, s.d_seq) != cudaSuccess)
            return set_error(s, "result copy launch failed");
        return true;
    };

    auto t0 = clock_type::now();
    const bool one_launch = fetch_by_kernel && !tensor_path && tokens <= chunk;
    if (one_launch) {
        // The whole call is one fixed chain of launches over fixed addresses: replay it from a graph.  The first call with a
        // given set of tensors runs the chain as plain launches (kernel attributes are set there, outside any capture),
        // the second captures it, every later one is a single cudaGraphLaunch.
        std::memcpy(s.h_input, x, x_bytes);
        s.stats.transfer_us += us_since(t0);
        t0 = clock_type::now();
        uint64_t key = 1469598103934665603ull;
        auto mix = [&key](uint64_t v) { key = (key ^ v) * 1099511628211ull; };
        for (size_t i = 0; i < count; ++i) mix(reinterpret_cast<uintptr_t>(w[i]));
        mix(tokens); mix(static_cast<uint64_t>(act_mode)); mix(count);
        auto it = s.use_host_graphs ? s.host_graphs.find(key) : s.host_graphs.end();
        if (it != s.host_graphs.end() && it->second.exec) {
            ZC_CUDA(s, cudaGraphLaunch(it->second.exec, s.stream));
            s.stats.dispatches += 3;
        } else if (it != s.host_graphs.end()) {
            cudaGraph_t graph = nullptr;
            ZC_CUDA(s, cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeThreadLocal));
            const bool ok = enqueue_chain();
            const cudaError_t e = cudaStreamEndCapture(s.stream, &graph);
            if (!ok || e != cudaSuccess || !graph) {
                if (graph) cudaGraphDestroy(graph);
                s.host_graphs.erase(it);
                s.use_host_graphs = false;          // this driver does not capture the chain: plain launches from now on
                if (ok) set_error(s, std::string("capturing the call failed: ") + cudaGetErrorString(e));
                cudaGetLastError();
                if (!enqueue_chain()) return false;
            } else {
                cudaGraphExec_t exec = nullptr;
                const cudaError_t ei = cudaGraphInstantiate(&exec, graph, 0);
                cudaGraphDestroy(graph);
                if (ei != cudaSuccess) return set_error(s, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(ei));
                it->second.exec = exec;
                ZC_CUDA(s, cudaGraphLaunch(exec, s.stream));
            }
        } else {
            if (s.use_host_graphs) {
                if (s.host_graphs.size() >= 4096) drop_host_graphs(s);
                s.host_graphs.emplace(key, State::HostGraph{});
            }
            if (!enqueue_chain()) return false;
        }
        s.stats.launch_us += us_since(t0);
        t0 = clock_type::now();
        if (!wait_done(s, ++s.done_seq)) return false;
    } else {
        if (fetch_by_kernel) {
            std::memcpy(s.h_input, x, x_bytes);
            const size_t n16 = x_bytes / sizeof(float4);
            stage_in_kernel<<<static_cast<unsigned>(std::min<size_t>((n16 + 255) / 256, 32)), 256, 0, s.stream>>>(
                reinterpret_cast<float4*>(s.d_x), reinterpret_cast<const float4*>(s.d_input), n16);
            ++s.stats.dispatches;
            if (cudaGetLastError() != cudaSuccess) return set_error(s, "activation fetch launch failed");
        } else {
            std::memcpy(s.h_stage, x, x_bytes);
            ZC_CUDA(s, cudaMemcpyAsync(s.d_x, s.h_stage, x_bytes, cudaMemcpyHostToDevice, s.stream));
        }
        s.stats.transfer_us += us_since(t0);
        t0 = clock_type::now();
        if (tensor_path && (fmt == ZEN_CUDA_Q4_K || fmt == ZEN_CUDA_Q5_K)) {
            size_t need = 0;
            for (size_t i = 0; i < count; ++i) need = std::max(need, gemm_k45_ws_bytes(tokens, rows[i], cols));
            if (!ensure_gemm_ws(s, need)) return false;
            for (size_t i = 0; i < count; ++i)
                if (!enqueue_gemm_k45(s, w[i], d_out[i], s.d_x, tokens, s.d_gemm_ws, s.stream, s.d_gemm_ws_bytes)) return false;
        } else if (tensor_path && fmt == ZEN_CUDA_Q4_0) {
            size_t need = 0;
            for (size_t i = 0; i < count; ++i) need = std::max(need, gemm_q4_0_ws_bytes(tokens, rows[i], cols));
            if (!ensure_gemm_ws(s, need)) return false;
            for (size_t i = 0; i < count; ++i)    // stream-ordered: the tensors share the scratch one after the other
                if (!enqueue_gemm_q4_0(s, w[i], d_out[i], s.d_x, tokens, s.d_gemm_ws, s.stream, s.d_gemm_ws_bytes)) return false;
        } else if (tensor_path && fmt == ZEN_CUDA_Q6_K) {
            if (!ensure_gemm_ws(s, gemm_q6k_ws_bytes(tokens, cols))) return false;
            for (size_t i = 0; i < count; ++i)    // stream-ordered: the tensors share the workspace one after the other
                if (!enqueue_gemm_q6k(s, w[i], d_out[i], s.d_x, tokens, s.d_gemm_ws, s.stream, s.d_gemm_ws_bytes)) return false;
        } else if (tensor_path) {
            if (!ensure_gemm_ws(s, gemm_ws_bytes_any(s, tokens, cols, act_mode))) return false;
            if (!enqueue_gemm_q8_0(s, w, d_out, count, s.d_x, tokens, s.d_gemm_ws, s.stream, act_mode, s.d_gemm_ws_bytes)) return false;
        }
        for (size_t t0k = 0; !tensor_path && t0k < tokens; t0k += chunk) {
            const size_t nt = std::min<size_t>(chunk, tokens - t0k);
            float* d_chunk[zk::kMaxTasks];
            for (size_t i = 0; i < count; ++i) d_chunk[i] = d_out[i] + t0k * rows[i];
            if (!enqueue_gemv(s, w, d_chunk, count, s.d_x + t0k * cols, nt, act_mode, s.stream)) return false;
        }
        s.stats.launch_us += us_since(t0);
        t0 = clock_type::now();
        if (direct) {
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(1);
            cfg.blockDim = dim3(1024);
            cfg.stream = s.stream;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr.val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = s.pdl ? 1 : 0;
            ++s.stats.dispatches;
            if (cudaLaunchKernelEx(&cfg, copy_out_publish_kernel, reinterpret_cast<float4*>(s.d_result), reinterpret_cast<const float4*>(s.d_y),
                                   (y_bytes + 15) / 16, s.d_done, s.d_seq) != cudaSuccess)
                return set_error(s, "result copy launch failed");
            if (!wait_done(s, ++s.done_seq)) return false;
        } else {
            ZC_CUDA(s, cudaMemcpyAsync(s.h_stage, s.d_y, y_bytes, cudaMemcpyDeviceToHost, s.stream));
            ZC_CUDA(s, cudaStreamSynchronize(s.stream));
        }
    }
    s.stats.wait_us += us_since(t0);
    if (!check_error_word(s)) return false;
    t0 = clock_type::now();
    off = 0;
    for (size_t i = 0; i < count; ++i) {
        std::memcpy(ys[i], reinterpret_cast<const uint8_t*>(h_result) + off * sizeof(float), tokens * rows[i] * sizeof(float));
        off += tokens * rows[i];
    }
    s.stats.readback_us += us_since(t0);
    ++s.stats.submits;
    if (count > 1) ++s.stats.batches;
    return true;
}

// ---- the two other host-pointer submissions of the backend contract ------------------------------------------------
// Both follow host_product's data path: small inputs are fetched from mapped host memory by a kernel and small results
// are stored to mapped host memory by the copy-out kernel; anything larger crosses on the copy engine.

// Lays `parts` (each padded to 16 bytes) end to end at the start of s.d_x.  offsets[i] receives part i's float offset.
bool host_fetch_parts(State& s, const void* const* parts, const size_t* bytes, size_t nparts, size_t* offsets, size_t y_bytes) {
    size_t total = 0;
    for (size_t i = 0; i < nparts; ++i) { offsets[i] = total / sizeof(float); total += (bytes[i] + 15) & ~size_t(15); }
    if (!ensure_scratch(s, total, y_bytes)) return false;
    const bool direct = y_bytes <= kDirectResultBytes;
    if (direct && !ensure_direct_result(s, y_bytes)) return false;
    const auto t0 = clock_type::now();
    const bool by_kernel = direct && total <= kDirectInputBytes;
    uint8_t* stage = reinterpret_cast<uint8_t*>(by_kernel ? s.h_input : s.h_stage);
    for (size_t i = 0; i < nparts; ++i) std::memcpy(stage + offsets[i] * sizeof(float), parts[i], bytes[i]);
    if (by_kernel) {
        const size_t n16 = total / sizeof(float4);
        stage_in_kernel<<<static_cast<unsigned>(std::min<size_t>((n16 + 255) / 256, 32)), 256, 0, s.stream>>>(
            reinterpret_cast<float4*>(s.d_x), reinterpret_cast<const float4*>(s.d_input), n16);
        ++s.stats.dispatches;
        if (cudaGetLastError() != cudaSuccess) return set_error(s, "activation fetch launch failed");
    } else {
        ZC_CUDA(s, cudaMemcpyAsync(s.d_x, s.h_stage, total, cudaMemcpyHostToDevice, s.stream));
    }
    s.stats.transfer_us += us_since(t0);
    return true;
}

// Brings the first y_bytes of s.d_y to `y` and finishes the call (error word, counters).
bool host_return(State& s, void* y, size_t y_bytes) {
    auto t0 = clock_type::now();
    const bool direct = y_bytes <= kDirectResultBytes;
    if (direct) {
        ++s.stats.dispatches;
        if (launch_pdl(s, copy_out_publish_kernel, dim3(1), dim3(1024), 0, s.stream, reinterpret_cast<float4*>(s.d_result),
                       reinterpret_cast<const float4*>(s.d_y), (y_bytes + 15) / 16, s.d_done, s.d_seq) != cudaSuccess)
            return set_error(s, "result copy launch failed");
        if (!wait_done(s, ++s.done_seq)) return false;
    } else {
        ZC_CUDA(s, cudaMemcpyAsync(s.h_stage, s.d_y, y_bytes, cudaMemcpyDeviceToHost, s.stream));
        ZC_CUDA(s, cudaStreamSynchronize(s.stream));
    }
    s.stats.wait_us += us_since(t0);
    if (!check_error_word(s)) return false;
    t0 = clock_type::now();
    std::memcpy(y, direct ? s.h_result : s.h_stage, y_bytes);
    s.stats.readback_us += us_since(t0);
    ++s.stats.submits;
    return true;
}

// zen::hip::rms_norm_locked, hip_backend.hip:724-776: y[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * weight, row by row.
bool host_rms_norm(State& s, const float* x, const float* weight, float* y, size_t rows, size_t cols, float eps) {
    if (!x || !weight || !y || !rows || !cols) return set_error(s, "rms_norm: bad arguments");
    if (rows > (size_t(1) << 31) / cols) return set_error(s, "rms_norm: too large");
    const size_t bytes = rows * cols * sizeof(float);
    const void* parts[2] = {x, weight};
    const size_t part_bytes[2] = {bytes, cols * sizeof(float)};
    size_t off[2];
    if (!host_fetch_parts(s, parts, part_bytes, 2, off, bytes)) return false;
    const auto t0 = clock_type::now();
    for (size_t r0 = 0; r0 < rows; r0 += 65535) {
        const size_t nr = std::min<size_t>(65535, rows - r0);
        const cudaError_t e = launch_pdl(s, zk::residual_rms_norm_kernel, dim3(static_cast<unsigned>(nr)), dim3(zk::kNormThreads), 0, s.stream,
                                         s.d_x + off[0] + r0 * cols, static_cast<const float*>(nullptr), static_cast<const float*>(s.d_x + off[1]),
                                         s.d_y + r0 * cols, static_cast<uint32_t>(cols), eps);
        if (e != cudaSuccess) return set_error(s, std::string("rms_norm launch: ") + cudaGetErrorString(e));
        ++s.stats.dispatches;
    }
    s.stats.launch_us += us_since(t0);
    return host_return(s, y, bytes);
}

// zen::hip::gemv_ffn_locked, hip_backend.hip:778-870: y = down * (silu(gate * x) * (up * x)) as one submission, the
// intermediate activation never leaving the device.  Two launches here: gate|up share one, and the down projection
// applies silu(g) * u while it loads its activations.
bool host_ffn(State& s, const uint8_t* gate, const uint8_t* up, const uint8_t* down, const float* x, float* y,
              size_t ffn_rows, size_t cols, size_t out_rows) {
    if (!gate || !up || !down || !x || !y || !ffn_rows || !out_rows || !cols) return set_error(s, "gemv_q8_0_ffn: bad arguments");
    if (cols % 32 || ffn_rows % 32) return set_error(s, "gemv_q8_0_ffn: widths are not block aligned");
    // all three resolved before anything is queued; a pass that evicted is repeated once
    const zen_cuda_weights* w[3];
    for (int pass = 0;; ++pass) {
        const uint64_t before = s.evictions;
        w[0] = lookup_locked(s, ZEN_CUDA_Q8_0, gate, ffn_rows, cols);
        w[1] = w[0] ? lookup_locked(s, ZEN_CUDA_Q8_0, up, ffn_rows, cols) : nullptr;
        w[2] = w[1] ? lookup_locked(s, ZEN_CUDA_Q8_0, down, out_rows, ffn_rows) : nullptr;
        if (!w[2]) return false;
        if (s.evictions == before) break;
        if (pass) return set_error(s, "the tensors of one submission do not fit the residency budget together");
    }
    const int mode = s.q8_act_mode;
    if (!max_tokens_per_launch(s, ZEN_CUDA_Q8_0, cols, mode) || !max_tokens_per_launch(s, ZEN_CUDA_Q8_0, ffn_rows, mode))
        return set_error(s, "gemv_q8_0_ffn: one activation row does not fit shared memory");
    const size_t out_pad = (out_rows + 63) & ~size_t(63);   // the result first (the copy-out kernel reads the start of the buffer)
    const void* parts[1] = {x};
    const size_t part_bytes[1] = {cols * sizeof(float)};
    size_t off[1];
    if (!host_fetch_parts(s, parts, part_bytes, 1, off, (out_pad + 2 * ffn_rows) * sizeof(float))) return false;
    const auto t0 = clock_type::now();
    float* d_gate_up[2] = {s.d_y + out_pad, s.d_y + out_pad + ffn_rows};
    float* d_out[1] = {s.d_y};
    if (!enqueue_gemv(s, w, d_gate_up, 2, s.d_x, 1, mode, s.stream)) return false;
    if (!enqueue_gemv(s, w + 2, d_out, 1, d_gate_up[1], 1, mode, s.stream, nullptr, d_gate_up[0])) return false;
    s.stats.launch_us += us_since(t0);
    if (!host_return(s, y, out_rows * sizeof(float))) return false;
    ++s.stats.batches;
    return true;
}

}  // namespace

extern "C" {

int zen_cuda_enabled(void) {
    if (opted_out()) return 0;
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    return init_locked(s) ? 1 : 0;
}

int zen_cuda_init(void) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    return init_locked(s) ? 1 : 0;
}

void zen_cuda_shutdown(void) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (s.ready) {
        cudaSetDevice(s.device);
        cudaStreamSynchronize(s.stream);
        cudaStreamSynchronize(s.copy_stream);
        drop_host_graphs(s);
        if (s.d_seq) cudaFree(s.d_seq);
        s.d_seq = nullptr;
        for (auto& kv : s.resident) free_weights(s, kv.second);
        s.resident.clear();
        if (s.d_x) cudaFree(s.d_x);
        if (s.d_y) cudaFree(s.d_y);
        if (s.d_gemm_ws) cudaFree(s.d_gemm_ws);
        s.d_gemm_ws = nullptr; s.d_gemm_ws_bytes = 0;
        if (s.h_stage) cudaFreeHost(s.h_stage);
        if (s.h_error) cudaFreeHost(s.h_error);
        if (s.h_result) cudaFreeHost(s.h_result);
        if (s.h_input) cudaFreeHost(s.h_input);
        s.h_input = s.d_input = nullptr;
        if (s.h_done) cudaFreeHost(const_cast<unsigned*>(s.h_done));
        s.h_result = s.d_result = nullptr; s.h_result_bytes = 0;
        s.h_done = nullptr; s.d_done = nullptr;
        for (int i = 0; i < 2; ++i) {
            if (s.bounce[i]) cudaFreeHost(s.bounce[i]);
            if (s.bounce_free[i]) cudaEventDestroy(s.bounce_free[i]);
            s.bounce[i] = nullptr; s.bounce_free[i] = nullptr;
        }
        if (s.stream) cudaStreamDestroy(s.stream);
        if (s.copy_stream) cudaStreamDestroy(s.copy_stream);
        s.d_x = s.d_y = nullptr; s.h_stage = nullptr; s.h_error = s.d_error = nullptr;
        s.d_x_bytes = s.d_y_bytes = s.h_stage_bytes = 0;
        s.stream = s.copy_stream = nullptr;
    }
    s.ready = false;
    s.failed = false;  // a failed init is latched only until shutdown (hip_backend.hip:921-923)
}

int zen_cuda_info(zen_cuda_adapter_info* out) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.ready || !out) return 0;
    *out = s.adapter;
    return 1;
}

void zen_cuda_get_stats(zen_cuda_stats* out) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (out) *out = s.stats;
}

const char* zen_cuda_last_error(void) {
    static thread_local std::string copy;
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    copy = s.last_error;
    return copy.c_str();
}

int zen_cuda_set_q8_act_mode(int mode) {
    if (mode != ZEN_CUDA_ACT_INT8 && mode != ZEN_CUDA_ACT_FP32) return 0;
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    s.q8_act_mode = mode;
    return 1;
}
int zen_cuda_get_q8_act_mode(void) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    return s.q8_act_mode;
}

int zen_cuda_gemv_q8_0(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_product(s, ZEN_CUDA_Q8_0, x, &weights, &y, &rows, 1, 1, columns, s.q8_act_mode) ? 1 : 0;
}

int zen_cuda_gemm_q8_0(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_product(s, ZEN_CUDA_Q8_0, input, &weights, &output, &rows, 1, tokens, columns, s.q8_act_mode) ? 1 : 0;
}

int zen_cuda_gemv_q8_0_batch(const float* x, const zen_cuda_gemv_task* tasks, size_t count) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!tasks || !count || count > ZEN_CUDA_MAX_BATCH) return set_error(s, "gemv_q8_0_batch: bad task list") ? 1 : 0;
    const uint8_t* w[ZEN_CUDA_MAX_BATCH]; float* y[ZEN_CUDA_MAX_BATCH]; size_t r[ZEN_CUDA_MAX_BATCH];
    for (size_t i = 0; i < count; ++i) {
        if (tasks[i].columns != tasks[0].columns) return set_error(s, "gemv_q8_0_batch: tasks must share columns") ? 1 : 0;
        w[i] = tasks[i].weights; y[i] = tasks[i].y; r[i] = tasks[i].rows;
    }
    return host_product(s, ZEN_CUDA_Q8_0, x, w, y, r, count, 1, tasks[0].columns, s.q8_act_mode) ? 1 : 0;
}

int zen_cuda_gemm_q8_0_batch(const float* x, const zen_cuda_gemm_task* tasks, size_t count, size_t tokens, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!tasks || !count || count > ZEN_CUDA_MAX_BATCH) return set_error(s, "gemm_q8_0_batch: bad task list") ? 1 : 0;
    const uint8_t* w[ZEN_CUDA_MAX_BATCH]; float* y[ZEN_CUDA_MAX_BATCH]; size_t r[ZEN_CUDA_MAX_BATCH];
    for (size_t i = 0; i < count; ++i) { w[i] = tasks[i].weights; y[i] = tasks[i].y; r[i] = tasks[i].rows; }
    return host_product(s, ZEN_CUDA_Q8_0, x, w, y, r, count, tokens, columns, s.q8_act_mode) ? 1 : 0;
}

int zen_cuda_gemm_q6_k(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_product(s, ZEN_CUDA_Q6_K, input, &weights, &output, &rows, 1, tokens, columns, ZEN_CUDA_ACT_FP32) ? 1 : 0;
}

int zen_cuda_gemm_q4_0(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_product(s, ZEN_CUDA_Q4_0, input, &weights, &output, &rows, 1, tokens, columns, ZEN_CUDA_ACT_FP32) ? 1 : 0;
}

int zen_cuda_gemm_kquant(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns, int q5) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_product(s, q5 ? ZEN_CUDA_Q5_K : ZEN_CUDA_Q4_K, input, &weights, &output, &rows, 1, tokens, columns, ZEN_CUDA_ACT_FP32) ? 1 : 0;
}

/* ---- the backend contract's two fused submissions and the residency budget ---- */
int zen_cuda_rms_norm(const float* x, const float* weight, float* y, size_t rows, size_t columns, float epsilon) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_rms_norm(s, x, weight, y, rows, columns, epsilon) ? 1 : 0;
}

int zen_cuda_gemv_q8_0_ffn(const uint8_t* gate, const uint8_t* up, const uint8_t* down, const float* x, float* y, size_t ffn_rows,
                           size_t columns, size_t out_rows) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    return host_ffn(s, gate, up, down, x, y, ffn_rows, columns, out_rows) ? 1 : 0;
}

int zen_cuda_set_q6k_codes(int on) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return -1;
    const int before = s.q6k_codes ? 1 : 0;
    s.q6k_codes = on != 0;
    return before;
}

int zen_cuda_set_gemm_groups(int on) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return -1;
    const int before = s.gemm_groups ? 1 : 0;
    s.gemm_groups = on != 0;
    return before;
}

int zen_cuda_set_vram_budget(uint64_t bytes) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    s.vram_budget = bytes ? bytes : default_vram_budget(s);
    return 1;
}

int zen_cuda_residency(uint64_t* budget_bytes, uint64_t* held_bytes, uint64_t* tensors, uint64_t* evictions) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.ready) return 0;
    if (budget_bytes) *budget_bytes = s.vram_budget;
    if (held_bytes) *held_bytes = s.stats.weight_bytes;
    if (tensors) *tensors = s.resident.size();
    if (evictions) *evictions = s.evictions;
    return 1;
}

void zen_cuda_release_weights(const uint8_t* weights) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.ready) return;
    cudaStreamSynchronize(s.stream);
    drop_host_graphs(s);   // a captured call may name the tensor that goes away
    for (auto it = s.resident.begin(); it != s.resident.end();) {
        if (it->first.ptr == weights) { free_weights(s, it->second); it = s.resident.erase(it); }
        else ++it;
    }
}

int zen_cuda_quantize_acts(const float* x, int8_t* codes, float* scales, size_t tokens, size_t columns) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!x || !codes || !scales || !tokens || !columns || columns % 32) return set_error(s, "quantize_acts: bad arguments") ? 1 : 0;
    const size_t n = tokens * columns, nblk = n / 32;
    const size_t scales_at = (n + 255) & ~size_t(255);  // scales follow the codes in the output scratch
    if (!ensure_scratch(s, n * sizeof(float), scales_at + nblk * sizeof(float))) return 0;
    int8_t* d_codes = reinterpret_cast<int8_t*>(s.d_y);
    float* d_scales = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s.d_y) + scales_at);
    std::memcpy(s.h_stage, x, n * sizeof(float));
    if (cudaMemcpyAsync(s.d_x, s.h_stage, n * sizeof(float), cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return set_error(s, "quantize_acts: copy failed") ? 1 : 0;
    zk::quantize_acts_kernel<<<static_cast<unsigned>((nblk + 7) / 8), 256, 0, s.stream>>>(s.d_x, d_codes, d_scales, nullptr, nblk);
    ++s.stats.dispatches;
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "quantize_acts: launch failed") ? 1 : 0;
    if (cudaMemcpyAsync(codes, d_codes, n, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess ||
        cudaMemcpyAsync(scales, d_scales, nblk * sizeof(float), cudaMemcpyDeviceToHost, s.stream) != cudaSuccess ||
        cudaStreamSynchronize(s.stream) != cudaSuccess)
        return set_error(s, "quantize_acts: readback failed") ? 1 : 0;
    ++s.stats.submits;
    return 1;
}

zen_cuda_weights* zen_cuda_dev_upload(int format, const uint8_t* weights, size_t rows_total, size_t columns, size_t first_row, size_t nrows) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return nullptr;
    return upload_locked(s, format, weights, rows_total, columns, first_row, nrows);
}

void zen_cuda_dev_free(zen_cuda_weights* w) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.ready || !w) return;
    cudaDeviceSynchronize();
    free_weights(s, w);
}

size_t zen_cuda_dev_weight_bytes(const zen_cuda_weights* w) { return w ? w->device_bytes : 0; }

int zen_cuda_dev_gemv(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x, size_t tokens,
                      int act_mode, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_y) return set_error(s, "dev_gemv: bad arguments") ? 1 : 0;
    return enqueue_gemv(s, w, d_y, count, d_x, tokens, act_mode, stream ? static_cast<cudaStream_t>(stream) : s.stream) ? 1 : 0;
}

int zen_cuda_dev_gemv_swiglu(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_gate, const float* d_up,
                             size_t tokens, int act_mode, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_y || !d_gate || !d_up) return set_error(s, "dev_gemv_swiglu: bad arguments") ? 1 : 0;
    return enqueue_gemv(s, w, d_y, count, d_up, tokens, act_mode, stream ? static_cast<cudaStream_t>(stream) : s.stream, nullptr, d_gate) ? 1 : 0;
}

int zen_cuda_dev_gemv_fused(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x, size_t tokens, int act_mode,
                            const zen_cuda_gemv_fusion* fusion, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_y || !d_x || !fusion) return set_error(s, "dev_gemv_fused: bad arguments") ? 1 : 0;
    return enqueue_gemv(s, w, d_y, count, d_x, tokens, act_mode, stream ? static_cast<cudaStream_t>(stream) : s.stream, nullptr, fusion->gate,
                        fusion->norm_weight, fusion->norm_eps, fusion->accumulate != 0, fusion->warm_next, fusion->swiglu_pair != 0) ? 1 : 0;
}

zen_cuda_gemv_list* zen_cuda_gemv_list_create(const zen_cuda_gemv_list_item* items, size_t count, int act_mode) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return nullptr;
    return list_create_locked(s, items, count, act_mode);
}

void zen_cuda_gemv_list_destroy(zen_cuda_gemv_list* list) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!list) return;
    if (s.ready) { cudaDeviceSynchronize(); cudaFree(list->d_counter); }
    delete list;
}

uint64_t zen_cuda_gemv_list_bytes(const zen_cuda_gemv_list* list) { return list ? list->algorithmic_bytes : 0; }

int zen_cuda_dev_gemv_list(const zen_cuda_gemv_list* list, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!list) return set_error(s, "dev_gemv_list: bad arguments") ? 1 : 0;
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : s.stream;
    // The items travel as kernel parameters: a long list goes out in pieces of zk::kListMaxItems, which stream order
    // chains (a piece's first item then waits for the whole piece before it, as any launch does).
    for (size_t first = 0; first < list->items.size(); first += zk::kListMaxItems) {
        const size_t n = std::min<size_t>(zk::kListMaxItems, list->items.size() - first);
        const cudaError_t e = n <= static_cast<size_t>(zk::kListFewItems) ? launch_list_piece<zk::kListFewItems>(s, *list, first, n, st)
                                                                          : launch_list_piece<zk::kListMaxItems>(s, *list, first, n, st);
        if (e != cudaSuccess) return set_error(s, std::string("dev_gemv_list launch: ") + cudaGetErrorString(e)) ? 1 : 0;
        ++s.stats.dispatches;
    }
    return 1;
}

size_t zen_cuda_gemm_workspace_bytes(size_t tokens, size_t columns) { return gemm_ws_bytes_any(state(), tokens, columns, ZEN_CUDA_ACT_INT8); }
size_t zen_cuda_gemm_workspace_bytes_act(size_t tokens, size_t columns, int act_mode) { return gemm_ws_bytes_any(state(), tokens, columns, act_mode); }

int zen_cuda_dev_gemm_q8_0_act(const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x, size_t tokens, int act_mode,
                               void* workspace, size_t workspace_bytes, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_out || !count || count > ZEN_CUDA_MAX_BATCH || !w[0]) return set_error(s, "dev_gemm: bad arguments") ? 1 : 0;
    if (act_mode != ZEN_CUDA_ACT_INT8 && act_mode != ZEN_CUDA_ACT_FP32) return set_error(s, "dev_gemm: bad activation mode") ? 1 : 0;
    if (workspace_bytes < gemm_ws_bytes(tokens, w[0]->cols, act_mode == ZEN_CUDA_ACT_FP32 ? 2 : 1)) return set_error(s, "dev_gemm: workspace too small") ? 1 : 0;
    return enqueue_gemm_q8_0(s, w, d_out, count, d_x, tokens, static_cast<uint8_t*>(workspace), stream ? static_cast<cudaStream_t>(stream) : s.stream,
                             act_mode, workspace_bytes) ? 1 : 0;
}

int zen_cuda_dev_gemm_q8_0(const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x, size_t tokens,
                           void* workspace, size_t workspace_bytes, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_out || !count || count > ZEN_CUDA_MAX_BATCH || !w[0]) return set_error(s, "dev_gemm: bad arguments") ? 1 : 0;
    if (workspace_bytes < gemm_ws_bytes(tokens, w[0]->cols)) return set_error(s, "dev_gemm: workspace too small") ? 1 : 0;
    return enqueue_gemm_q8_0(s, w, d_out, count, d_x, tokens, static_cast<uint8_t*>(workspace),
                             stream ? static_cast<cudaStream_t>(stream) : s.stream, ZEN_CUDA_ACT_INT8, workspace_bytes) ? 1 : 0;
}

size_t zen_cuda_gemm_q6_k_workspace_bytes(size_t tokens, size_t columns) { return gemm_q6k_ws_bytes(tokens, columns); }

size_t zen_cuda_gemm_q4_0_workspace_bytes(size_t tokens, size_t rows, size_t columns) { return gemm_q4_0_ws_bytes(tokens, rows, columns); }

size_t zen_cuda_gemm_kquant_workspace_bytes(size_t tokens, size_t rows, size_t columns) { return gemm_k45_ws_bytes(tokens, rows, columns); }

int zen_cuda_dev_gemm_kquant(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace, size_t workspace_bytes,
                             void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_out || !d_x || !tokens) return set_error(s, "dev_gemm_kquant: bad arguments") ? 1 : 0;
    if (w->format != ZEN_CUDA_Q4_K && w->format != ZEN_CUDA_Q5_K) return set_error(s, "dev_gemm_kquant: a Q4_K or Q5_K tensor") ? 1 : 0;
    if (workspace_bytes < gemm_k45_ws_bytes(tokens, w->rows, w->cols)) return set_error(s, "dev_gemm_kquant: workspace too small") ? 1 : 0;
    return enqueue_gemm_k45(s, w, d_out, d_x, tokens, static_cast<uint8_t*>(workspace), stream ? static_cast<cudaStream_t>(stream) : s.stream, workspace_bytes) ? 1 : 0;
}

int zen_cuda_dev_gemm_q4_0(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace, size_t workspace_bytes,
                           void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_out || !d_x || !tokens) return set_error(s, "dev_gemm_q4_0: bad arguments") ? 1 : 0;
    if (w->format != ZEN_CUDA_Q4_0 || w->cols % 128) return set_error(s, "dev_gemm_q4_0: a Q4_0 tensor whose columns are a multiple of 128") ? 1 : 0;
    if (workspace_bytes < gemm_q4_0_ws_bytes(tokens, w->rows, w->cols)) return set_error(s, "dev_gemm_q4_0: workspace too small") ? 1 : 0;
    return enqueue_gemm_q4_0(s, w, d_out, d_x, tokens, static_cast<uint8_t*>(workspace), stream ? static_cast<cudaStream_t>(stream) : s.stream, workspace_bytes) ? 1 : 0;
}

int zen_cuda_dev_gemm_q6_k(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace, size_t workspace_bytes,
                           void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!w || !d_out || !d_x || !tokens) return set_error(s, "dev_gemm_q6_k: bad arguments") ? 1 : 0;
    if (w->format != ZEN_CUDA_Q6_K) return set_error(s, "dev_gemm_q6_k: not a Q6_K tensor") ? 1 : 0;
    if (workspace_bytes < gemm_q6k_ws_bytes(tokens, w->cols)) return set_error(s, "dev_gemm_q6_k: workspace too small") ? 1 : 0;
    return enqueue_gemm_q6k(s, w, d_out, d_x, tokens, static_cast<uint8_t*>(workspace), stream ? static_cast<cudaStream_t>(stream) : s.stream, workspace_bytes) ? 1 : 0;
}

int zen_cuda_dev_gemm_q8_0_noalloc(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    // No lazy initialisation here: that would allocate.  A resident tensor implies a ready backend.
    if (!s.ready) return set_error(s, "noalloc: backend not initialised; upload the tensor first") ? 1 : 0;
    if (!w || !d_out || !d_x || !tokens) return set_error(s, "noalloc: bad arguments") ? 1 : 0;
    if (w->format != ZEN_CUDA_Q8_0) return set_error(s, "noalloc: Q8_0 tensors only") ? 1 : 0;
    if (tokens > ZEN_CUDA_NOALLOC_MAX_ACT_ELEMENTS / w->cols || gemm_ws_bytes(tokens, w->cols) > ZEN_CUDA_NOALLOC_SCRATCH_BYTES)
        return set_error(s, "noalloc: tokens x columns = " + std::to_string(tokens * w->cols) + " exceeds the built-in scratch (" +
                                std::to_string(ZEN_CUDA_NOALLOC_MAX_ACT_ELEMENTS) + " activation elements); use zen_cuda_dev_gemm_q8_0 with a caller workspace") ? 1 : 0;
    uint8_t* scratch = nullptr;
    if (!noalloc_scratch_address(s, &scratch)) return 0;
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : s.stream;
    // The array still holds the previous call's bytes.  Codes of rows >= tokens are never read (the tensor map ends at
    // `tokens`), but the padded tail of every scale row is, so the scale area starts from zero.
    const size_t codes_bytes = (tokens * w->cols + 255) & ~size_t(255);
    const size_t scale_bytes = gemm_ws_bytes(tokens, w->cols) - codes_bytes;
    if (cudaMemsetAsync(scratch + codes_bytes, 0, scale_bytes, st) != cudaSuccess) return set_error(s, "noalloc: clearing the scale area failed") ? 1 : 0;
    const zen_cuda_weights* ws[1] = {w};
    float* outs[1] = {d_out};
    return enqueue_gemm_q8_0(s, ws, outs, 1, d_x, tokens, scratch, st) ? 1 : 0;
}

int zen_cuda_dev_quantize_acts(const float* d_x, int8_t* d_codes, float* d_scales, size_t tokens, size_t columns, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!d_x || !d_codes || !d_scales || !tokens || !columns || columns % 32) return set_error(s, "dev_quantize_acts: bad arguments") ? 1 : 0;
    const size_t nblk = tokens * columns / 32;
    zk::quantize_acts_kernel<<<static_cast<unsigned>((nblk + 7) / 8), 256, 0, stream ? static_cast<cudaStream_t>(stream) : s.stream>>>(
        d_x, d_codes, d_scales, nullptr, nblk);
    ++s.stats.dispatches;
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "dev_quantize_acts: launch failed") ? 1 : 0;
    return 1;
}

// ---- row-sharded products: gather regions shared between processes through CUDA IPC ------------------------------

size_t zen_cuda_gather_region_bytes(size_t world, size_t slot_floats) {
    if (!world || world > zk::kMaxPeers || !slot_floats) return 0;
    return zk::peer_region_bytes(world, slot_floats);
}

void* zen_cuda_ipc_alloc(size_t bytes, unsigned char handle_out[ZEN_CUDA_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == ZEN_CUDA_IPC_HANDLE_BYTES, "IPC handle size");
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return nullptr;
    if (!bytes || !handle_out) { set_error(s, "ipc_alloc: bad arguments"); return nullptr; }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h{};
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        set_error(s, std::string("ipc_alloc: ") + cudaGetErrorString(e));
        return nullptr;
    }
    std::memcpy(handle_out, &h, sizeof h);
    return p;
}

void* zen_cuda_ipc_open(const unsigned char handle[ZEN_CUDA_IPC_HANDLE_BYTES]) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return nullptr;
    if (!handle) { set_error(s, "ipc_open: bad arguments"); return nullptr; }
    cudaIpcMemHandle_t h{};
    std::memcpy(&h, handle, sizeof h);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_error(s, std::string("ipc_open: ") + cudaGetErrorString(e)); return nullptr; }
    return p;
}

void zen_cuda_ipc_close(void* peer_region) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (s.ready && peer_region) cudaIpcCloseMemHandle(peer_region);
}

void zen_cuda_ipc_free(void* own_region) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (s.ready && own_region) { cudaDeviceSynchronize(); cudaFree(own_region); }
}

zen_cuda_gather* zen_cuda_gather_create(size_t world, size_t rank, size_t slot_floats, void* const* regions) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return nullptr;
    if (!world || world > zk::kMaxPeers || rank >= world || !slot_floats || !regions) { set_error(s, "gather_create: bad arguments"); return nullptr; }
    for (size_t r = 0; r < world; ++r)
        if (!regions[r]) { set_error(s, "gather_create: a region is missing"); return nullptr; }
    auto* g = new zen_cuda_gather();
    if (cudaMalloc(&g->counters, 32) != cudaSuccess || cudaMemset(g->counters, 0, 32) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        if (g->counters) cudaFree(g->counters);
        delete g;
        set_error(s, "gather_create: out of device memory");
        return nullptr;
    }
    const size_t flag_offset = zk::peer_region_flag_offset(world, slot_floats);
    for (size_t r = 0; r < world; ++r) {
        g->dev.region[r] = static_cast<float*>(regions[r]);
        g->dev.flags[r] = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(regions[r]) + flag_offset);
    }
    g->dev.local_region = g->dev.region[rank];
    g->dev.local_flags = g->dev.flags[rank];
    g->dev.epoch = static_cast<unsigned long long*>(g->counters);
    g->dev.arrive = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(g->counters) + 8);
    g->dev.published = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(g->counters) + 16);
    g->dev.world = static_cast<uint32_t>(world);
    g->dev.rank = static_cast<uint32_t>(rank);
    g->dev.slot_floats = static_cast<uint32_t>(slot_floats);
    // The grid of every launch on this object: a function of the slot size alone, so all ranks agree whatever their shards.
    g->dev.grid = static_cast<uint32_t>(std::max<size_t>(1, std::min<size_t>((slot_floats + zk::kGemvWarps - 1) / zk::kGemvWarps, static_cast<size_t>(s.sm_count))));
    return g;
}

void zen_cuda_gather_destroy(zen_cuda_gather* g) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!g) return;
    if (s.ready) { cudaDeviceSynchronize(); cudaFree(g->counters); }
    delete g;
}

int zen_cuda_dev_gemv_gather(zen_cuda_gather* g, const zen_cuda_weights* const* w, float* const* d_y, size_t count,
                             const float* d_x, size_t tokens, int act_mode, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!g || !w) return set_error(s, "dev_gemv_gather: bad arguments") ? 1 : 0;
    return enqueue_gemv(s, w, d_y, count, d_x, tokens, act_mode, stream ? static_cast<cudaStream_t>(stream) : s.stream, &g->dev) ? 1 : 0;
}

int zen_cuda_dev_gather_fetch(zen_cuda_gather* g, float* d_out, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!g) return set_error(s, "dev_gather_fetch: bad arguments") ? 1 : 0;
    const size_t n = static_cast<size_t>(g->dev.world) * g->dev.slot_floats;
    const unsigned grid = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>((n + 1023) / 1024, static_cast<size_t>(s.sm_count))));
    zk::gather_fetch_kernel<<<grid, 256, 0, stream ? static_cast<cudaStream_t>(stream) : s.stream>>>(g->dev, d_out, s.d_error);
    ++s.stats.dispatches;
    if (cudaGetLastError() != cudaSuccess) return set_error(s, "dev_gather_fetch: launch failed") ? 1 : 0;
    return 1;
}

int zen_cuda_dev_allgather(zen_cuda_gather* g, const float* d_piece, size_t count, float* d_whole, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!g || !d_piece || !d_whole || !count || count % 4 || g->dev.slot_floats % 4 || count > g->dev.slot_floats ||
        (reinterpret_cast<uintptr_t>(d_piece) | reinterpret_cast<uintptr_t>(d_whole)) % 16)
        return set_error(s, "dev_allgather: bad arguments (count and slot: multiples of 4 floats, count <= slot, 16-byte aligned vectors)") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::allgather_kernel, dim3(1), dim3(1024), 0, stream ? static_cast<cudaStream_t>(stream) : s.stream, g->dev, d_piece,
                                     static_cast<uint32_t>(count), d_whole, s.d_error);
    ++s.stats.dispatches;
    if (e != cudaSuccess) return set_error(s, std::string("dev_allgather: launch failed: ") + cudaGetErrorString(e)) ? 1 : 0;
    return 1;
}

int zen_cuda_dev_allreduce_add(zen_cuda_gather* g, const float* d_partial, size_t count, float* d_inout, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!g || !d_partial || !d_inout || d_partial == d_inout || !count || count % 4 || g->dev.slot_floats % 4 || count > g->dev.slot_floats ||
        (reinterpret_cast<uintptr_t>(d_partial) | reinterpret_cast<uintptr_t>(d_inout)) % 16)
        return set_error(s, "dev_allreduce_add: bad arguments (count and slot: multiples of 4 floats, count <= slot, 16-byte aligned distinct vectors)") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::allreduce_add_kernel, dim3(1), dim3(1024), 0, stream ? static_cast<cudaStream_t>(stream) : s.stream, g->dev,
                                     d_partial, static_cast<uint32_t>(count), d_inout, s.d_error);
    ++s.stats.dispatches;
    if (e != cudaSuccess) return set_error(s, std::string("dev_allreduce_add: launch failed: ") + cudaGetErrorString(e)) ? 1 : 0;
    return 1;
}

int zen_cuda_dev_greedy_pick(const zen_cuda_pick_segment* segments, size_t count, size_t tokens, int64_t* d_pick, void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!segments || !count || count > zk::kPickMaxSegments || !tokens || tokens > 65535 || !d_pick) return set_error(s, "dev_greedy_pick: bad arguments") ? 1 : 0;
    zk::PickParams p{};
    size_t longest = 0;
    for (size_t i = 0; i < count; ++i) {
        if (!segments[i].base && segments[i].len) return set_error(s, "dev_greedy_pick: null segment") ? 1 : 0;
        if (static_cast<uint64_t>(segments[i].first_index) + segments[i].len > 0xffffffffull) return set_error(s, "dev_greedy_pick: index range too large") ? 1 : 0;
        p.seg[i] = zk::PickSegment{segments[i].base, segments[i].len, segments[i].first_index, segments[i].token_stride, 0};
        longest = std::max<size_t>(longest, segments[i].len);
    }
    p.nseg = static_cast<uint32_t>(count);
    // enough CTAs to fill the machine once, at least 2048 entries each
    const size_t want = std::max<size_t>(1, static_cast<size_t>(s.sm_count) * 2 / (count * tokens));
    p.ctas_per_segment = static_cast<uint32_t>(std::max<size_t>(1, std::min(want, (longest + 2047) / 2048)));
    p.keys = reinterpret_cast<unsigned long long*>(d_pick);
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : s.stream;
    ZC_CUDA(s, cudaMemsetAsync(d_pick, 0, tokens * sizeof(int64_t), st));
    cudaError_t e = launch_pdl(s, zk::pick_scan_kernel, dim3(p.nseg * p.ctas_per_segment, static_cast<unsigned>(tokens)), dim3(zk::kPickThreads), 0, st, p);
    if (e == cudaSuccess)
        e = launch_pdl(s, zk::pick_finish_kernel, dim3(static_cast<unsigned>((tokens + 63) / 64)), dim3(64), 0, st, p.keys, static_cast<uint32_t>(tokens));
    s.stats.dispatches += 2;
    if (e != cudaSuccess) return set_error(s, "dev_greedy_pick: launch failed") ? 1 : 0;
    return 1;
}

int zen_cuda_dev_sample(const float* d_logits, size_t n, float temperature, uint32_t top_k, float top_p, double u, int64_t* d_pick,
                        int32_t* d_kept_ids, double* d_kept_probs, int32_t* d_kept_count, int32_t* d_truncated, void* stream) {
    static_assert(ZEN_CUDA_SAMPLE_MAX_CANDIDATES == zk::kSampleMaxCandidates, "candidate limit");
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    if (!d_logits || !n || n > 0xffffffffull || !d_pick || !(temperature > 0.0f) || !std::isfinite(temperature) || !(u >= 0.0 && u < 1.0))
        return set_error(s, "dev_sample: bad arguments (temperature > 0, u in [0, 1))") ? 1 : 0;
    zk::SampleParams p{};
    p.logits = d_logits; p.n = static_cast<uint32_t>(n); p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.u = u;
    p.pick = reinterpret_cast<long long*>(d_pick); p.kept_ids = d_kept_ids; p.kept_probs = d_kept_probs; p.kept_count = d_kept_count; p.truncated = d_truncated;
    const cudaError_t e = launch_pdl(s, zk::sample_top_kernel, dim3(1), dim3(zk::kSampleThreads), 0, stream ? static_cast<cudaStream_t>(stream) : s.stream, p);
    ++s.stats.dispatches;
    if (e != cudaSuccess) return set_error(s, std::string("dev_sample: launch failed: ") + cudaGetErrorString(e)) ? 1 : 0;
    return 1;
}

// ---- decode-step operators ------------------------------------------------------------------------------------------

#define ZC_DEV_ENTER(name)                                   \
    State& s = state();                                      \
    std::lock_guard<std::mutex> lock(s.mutex);               \
    if (!init_locked(s)) return 0;                           \
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : s.stream; \
    const char* const entry_name = name;                     \
    (void)entry_name
#define ZC_DEV_LEAVE(launch_result)                                                                            \
    ++s.stats.dispatches;                                                                                      \
    if ((launch_result) != cudaSuccess) return set_error(s, std::string(entry_name) + ": launch failed") ? 1 : 0; \
    return 1

int zen_cuda_dev_embed_q8_0(const zen_cuda_weights* w, const int64_t* d_token, float* d_out, void* stream) {
    ZC_DEV_ENTER("dev_embed_q8_0");
    if (!w || !d_token || !d_out || w->format != ZEN_CUDA_Q8_0) return set_error(s, "dev_embed_q8_0: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::embed_row_q8_0_kernel, dim3(static_cast<unsigned>((w->cols + 255) / 256)), dim3(256), 0, st,
        static_cast<const int8_t*>(w->plane[0]), static_cast<const __half*>(w->plane[1]), static_cast<uint32_t>(w->rows), static_cast<uint32_t>(w->cols),
        w->nbp, reinterpret_cast<const long long*>(d_token), d_out, s.d_error);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_rms_norm(float* d_x, const float* d_delta, const float* d_weight, float* d_y, size_t n, size_t rows, float eps, void* stream) {
    ZC_DEV_ENTER("dev_rms_norm");
    if (!d_x || !n || !rows || rows > 65535 || (d_weight && !d_y) || (!d_weight && !d_delta)) return set_error(s, "dev_rms_norm: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::residual_rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(zk::kNormThreads), 0, st, d_x, d_delta, d_weight, d_y,
                                     static_cast<uint32_t>(n), eps);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_rope_kv_append(float* d_q, float* d_k, const float* d_v, const float* d_cos, const float* d_sin, const int* d_pos,
                                size_t heads, size_t kv_heads, size_t head_dim, size_t pairs, int adjacent, float* d_k_cache, float* d_v_cache,
                                size_t max_positions, void* stream) {
    ZC_DEV_ENTER("dev_rope_kv_append");
    if (!d_q || !d_k || !d_v || !d_cos || !d_sin || !d_pos || !d_k_cache || !d_v_cache || !heads || !kv_heads || !head_dim || 2 * pairs > head_dim ||
        !max_positions)
        return set_error(s, "dev_rope_kv_append: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::rope_kv_append_kernel, dim3(1), dim3(1024), 0, st, d_q, d_k, d_v, d_cos, d_sin, d_pos,
                                     static_cast<uint32_t>(heads), static_cast<uint32_t>(kv_heads), static_cast<uint32_t>(head_dim),
                                     static_cast<uint32_t>(pairs), adjacent, d_k_cache, d_v_cache, static_cast<uint32_t>(max_positions), s.d_error);
    ZC_DEV_LEAVE(e);
}

namespace {
// Shared by the two attention entry points.  fused: q/k/v are the raw projections, rope and the cache append happen inside.
bool enqueue_attention(State& s, cudaStream_t st, bool fused, const float* d_q, const float* d_k, const float* d_v, const float* d_cos, const float* d_sin,
                       size_t pairs, const int* d_pos, float* d_k_cache, float* d_v_cache, float* d_out, size_t heads, size_t kv_heads, size_t head_dim,
                       float scale, size_t window, size_t max_positions) {
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out || !heads || !kv_heads || heads % kv_heads || !head_dim || head_dim % 4 || head_dim > 256 ||
        !max_positions || (fused && (!d_k || !d_v || !d_cos || !d_sin || 2 * pairs > head_dim)))
        return set_error(s, "attention: bad arguments");
    const size_t smem = 0;   // the streaming softmax keeps no per-position scores
    if (scale == 0.0f) scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
    const dim3 grid(zk::kAttnSplit, static_cast<unsigned>(heads)), block(zk::kAttnThreads);
    const bool wide = head_dim > 128;
    auto launch = [&](auto kernel) {
        return fused ? launch_pdl(s, kernel, grid, block, smem, st, d_q, static_cast<const float*>(nullptr), static_cast<const float*>(nullptr), d_pos, d_out,
                                  static_cast<uint32_t>(heads), static_cast<uint32_t>(kv_heads), static_cast<uint32_t>(head_dim), scale, static_cast<uint32_t>(window),
                                  static_cast<uint32_t>(max_positions), s.d_error, d_k, d_v, d_cos, d_sin, static_cast<uint32_t>(pairs), d_k_cache, d_v_cache)
                     : launch_pdl(s, kernel, grid, block, smem, st, d_q, static_cast<const float*>(d_k_cache), static_cast<const float*>(d_v_cache), d_pos, d_out,
                                  static_cast<uint32_t>(heads), static_cast<uint32_t>(kv_heads), static_cast<uint32_t>(head_dim), scale, static_cast<uint32_t>(window),
                                  static_cast<uint32_t>(max_positions), s.d_error, static_cast<const float*>(nullptr), static_cast<const float*>(nullptr),
                                  static_cast<const float*>(nullptr), static_cast<const float*>(nullptr), 0u, static_cast<float*>(nullptr), static_cast<float*>(nullptr));
    };
    const cudaError_t e = fused ? (wide ? launch(zk::attention_decode_kernel<true, true>) : launch(zk::attention_decode_kernel<true, false>))
                                : (wide ? launch(zk::attention_decode_kernel<false, true>) : launch(zk::attention_decode_kernel<false, false>));
    ++s.stats.dispatches;
    if (e != cudaSuccess) return set_error(s, "attention: launch failed");
    return true;
}
}  // namespace

int zen_cuda_dev_attention(const float* d_q, const float* d_k_cache, const float* d_v_cache, const int* d_pos, float* d_out, size_t heads,
                           size_t kv_heads, size_t head_dim, float scale, size_t window, size_t max_positions, void* stream) {
    ZC_DEV_ENTER("dev_attention");
    return enqueue_attention(s, st, false, d_q, nullptr, nullptr, nullptr, nullptr, 0, d_pos, const_cast<float*>(d_k_cache), const_cast<float*>(d_v_cache), d_out,
                             heads, kv_heads, head_dim, scale, window, max_positions) ? 1 : 0;
}

int zen_cuda_dev_attention_block(const float* d_q, const float* d_k, const float* d_v, const float* d_cos, const float* d_sin, size_t pairs, const int* d_pos,
                                 float* d_k_cache, float* d_v_cache, float* d_out, size_t heads, size_t kv_heads, size_t head_dim, float scale, size_t window,
                                 size_t max_positions, void* stream) {
    ZC_DEV_ENTER("dev_attention_block");
    return enqueue_attention(s, st, true, d_q, d_k, d_v, d_cos, d_sin, pairs, d_pos, d_k_cache, d_v_cache, d_out, heads, kv_heads, head_dim, scale, window,
                             max_positions) ? 1 : 0;
}

int zen_cuda_dev_embed_rows_q8_0(const zen_cuda_weights* w, const int64_t* d_tokens, size_t tokens, float* d_out, void* stream) {
    ZC_DEV_ENTER("dev_embed_rows_q8_0");
    if (!w || !d_tokens || !tokens || tokens > 65535 || !d_out || w->format != ZEN_CUDA_Q8_0) return set_error(s, "dev_embed_rows_q8_0: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::embed_rows_q8_0_kernel, dim3(static_cast<unsigned>((w->cols + 255) / 256), static_cast<unsigned>(tokens)), dim3(256), 0, st,
        static_cast<const int8_t*>(w->plane[0]), static_cast<const __half*>(w->plane[1]), static_cast<uint32_t>(w->rows), static_cast<uint32_t>(w->cols),
        w->nbp, reinterpret_cast<const long long*>(d_tokens), d_out, s.d_error);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_rope_kv_append_rows(float* d_q, float* d_k, const float* d_v, size_t tokens, const float* d_cos, const float* d_sin, const int* d_pos,
                                     size_t heads, size_t kv_heads, size_t head_dim, size_t pairs, int adjacent, float* d_k_cache, float* d_v_cache,
                                     size_t max_positions, void* stream) {
    ZC_DEV_ENTER("dev_rope_kv_append_rows");
    if (!d_q || !d_k || !d_v || !tokens || tokens > 65535 || !d_cos || !d_sin || !d_pos || !d_k_cache || !d_v_cache || !heads || !kv_heads || !head_dim ||
        2 * pairs > head_dim || !max_positions)
        return set_error(s, "dev_rope_kv_append_rows: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::rope_kv_append_rows_kernel, dim3(static_cast<unsigned>(tokens)), dim3(1024), 0, st, d_q, d_k, d_v, d_cos, d_sin, d_pos,
                                     static_cast<uint32_t>(heads), static_cast<uint32_t>(kv_heads), static_cast<uint32_t>(head_dim),
                                     static_cast<uint32_t>(pairs), adjacent, d_k_cache, d_v_cache, static_cast<uint32_t>(max_positions), s.d_error);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_attention_prefill(const float* d_q, const float* d_k_cache, const float* d_v_cache, const int* d_pos, float* d_out, size_t tokens,
                                   size_t heads, size_t kv_heads, size_t head_dim, float scale, size_t window, size_t max_positions, void* stream) {
    ZC_DEV_ENTER("dev_attention_prefill");
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out || !tokens || !heads || !kv_heads || heads % kv_heads || kv_heads > 65535 || !max_positions ||
        (head_dim != 64 && head_dim != 128 && head_dim != 256))
        return set_error(s, "dev_attention_prefill: bad arguments (head_dim 64, 128 or 256)") ? 1 : 0;
    if (scale == 0.0f) scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
    // query heads per thread: the largest of 4, 2, 1 that divides the group and keeps 2 * R * head_dim / 8 row values in registers
    const size_t group = heads / kv_heads;
    const int cap = head_dim == 256 ? 2 : 4;
    const int r_heads = (cap >= 4 && group % 4 == 0) ? 4 : (group % 2 == 0) ? 2 : 1;
    const size_t n_tiles = (tokens + zk::kPfTokens - 1) / zk::kPfTokens, n_ctas = n_tiles * kv_heads * (group / r_heads);
    if (n_ctas > 0x7fffffffu) return set_error(s, "dev_attention_prefill: too many tiles") ? 1 : 0;
    const dim3 grid(static_cast<unsigned>(n_ctas)), block(zk::kPfThreads);
    const size_t smem = 2 * 2 * zk::kPfBlock * head_dim * sizeof(float);   // two buffers of keys + values
    auto launch = [&](auto kernel) {
        // the instantiations share one function-pointer type, so the opt-in flags are keyed by (head_dim, heads per thread)
        static bool configured[3][3] = {};
        bool& done = configured[head_dim == 64 ? 0 : head_dim == 128 ? 1 : 2][r_heads == 4 ? 2 : r_heads == 2 ? 1 : 0];
        if (!done && smem > 48 * 1024) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return cudaErrorInvalidValue;
            done = true;
        }
        return launch_pdl(s, kernel, grid, block, smem, st, d_q, d_k_cache, d_v_cache, d_pos, d_out, static_cast<uint32_t>(tokens), static_cast<uint32_t>(heads),
                          static_cast<uint32_t>(kv_heads), scale, static_cast<uint32_t>(window), static_cast<uint32_t>(max_positions), s.d_error);
    };
    auto by_heads = [&](auto dim) {
        constexpr int kD = decltype(dim)::value;
        if constexpr (kD < 256) {
            if (r_heads == 4) return launch(zk::attention_prefill_kernel<kD, 4>);
        }
        return r_heads == 2 ? launch(zk::attention_prefill_kernel<kD, 2>) : launch(zk::attention_prefill_kernel<kD, 1>);
    };
    const cudaError_t e = head_dim == 64 ? by_heads(std::integral_constant<int, 64>{}) : head_dim == 128 ? by_heads(std::integral_constant<int, 128>{})
                                                                                                          : by_heads(std::integral_constant<int, 256>{});
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_silu_mul(const float* d_gate, const float* d_up, float* d_out, size_t count, void* stream) {
    ZC_DEV_ENTER("dev_silu_mul");
    if (!d_gate || !d_up || !d_out || !count) return set_error(s, "dev_silu_mul: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::silu_mul_kernel, dim3(static_cast<unsigned>(std::min<size_t>((count + 255) / 256, 4 * static_cast<size_t>(s.sm_count)))),
                                     dim3(256), 0, st, d_gate, d_up, d_out, count);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_advance_position(int* d_pos, int delta, void* stream) {
    ZC_DEV_ENTER("dev_advance_position");
    if (!d_pos) return set_error(s, "dev_advance_position: bad arguments") ? 1 : 0;
    const cudaError_t e = launch_pdl(s, zk::advance_position_kernel, dim3(1), dim3(1), 0, st, d_pos, delta);
    ZC_DEV_LEAVE(e);
}

int zen_cuda_dev_check(void* stream) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.ready) { set_error(s, "dev_check: backend not initialised"); return -1; }
    cudaError_t e = cudaStreamSynchronize(stream ? static_cast<cudaStream_t>(stream) : s.stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {   // a failed launch or a fault: not one of the kernels' own codes
        set_error(s, std::string("dev_check: ") + cudaGetErrorString(e));
        return -static_cast<int>(e) - 1;
    }
    const int code = *s.h_error;
    *s.h_error = 0;
    if (code) set_error(s, std::string("device-side error word: ") + zen_cuda_error_name(code));
    return code;
}

const char* zen_cuda_error_name(int code) {
    switch (code) {
    case 0: return "none";
    case zk::kErrFullWaitTimeout: return "wait for a weight stage to land timed out";
    case zk::kErrEmptyWaitTimeout: return "wait for a free weight stage timed out";
    case zk::kErrDrainTimeout: return "wait for copies in flight at kernel exit timed out";
    case zk::kErrTmemWaitTimeout: return "wait for a tensor-memory accumulator timed out";
    case zk::kErrPeerWaitTimeout: return "a peer GPU did not publish its outputs in time";
    case zk::kErrBadToken: return "token id outside the embedding table";
    case zk::kErrBadPosition: return "position outside the KV cache";
    case zk::kErrNonFinite: return "non-finite value in attention";
    case zk::kErrInputWaitTimeout: return "wait for a work-list item's input timed out";
    default: return code < 0 ? "CUDA runtime error (see zen_cuda_last_error)" : "unknown";
    }
}

int zen_cuda_set_wait_budget_ms(unsigned milliseconds) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!init_locked(s)) return 0;
    ZC_CUDA(s, cudaStreamSynchronize(s.stream));
    return apply_wait_budget(s, milliseconds) ? 1 : 0;
}

#ifdef ZK_TRACE
__attribute__((visibility("default"))) void zen_cuda_debug_trace(void* dev, size_t start) { g_trace = static_cast<unsigned long long*>(dev); g_trace_launch = start; }
#endif

}  // extern "C"
