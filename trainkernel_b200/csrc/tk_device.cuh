// Device-side building blocks of the generated sm_100a training-step kernel.
//
// The generator emits one persistent cooperative kernel per program and glues
// these pieces together: a hand-written grid barrier, a warp-specialised
// tcgen05 GEMM pipeline (TMA -> swizzled shared memory -> tcgen05.mma -> TMEM ->
// tcgen05.ld epilogue), an exact-FP32 SIMT GEMM, a GEMV, and row helpers used
// by the generated pointwise / reduction / epilogue code.
//
// Every wait in this file is bounded by a wall-clock limit.  When a limit is
// hit the kernel records {code, stage, block, detail} in the status words,
// raises a block-wide and grid-wide abort flag, skips the remaining work and
// returns normally, so the CUDA context stays usable and the host can report.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <type_traits>

namespace tk {

constexpr int kThreads = 192;          // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
// Epilogue warps of the cta_group::1 GEMM: 4 (warps 2..5), or 8 in a kernel generated with the wide epilogue
// (320 threads: warps 6..9 read the same TMEM quarters as warps 2..5 and take every other 32-column chunk; they
// do nothing outside tensor-core GEMM units).  A generated kernel defines TK_EPI_WARPS before including this file.
#ifndef TK_EPI_WARPS
#define TK_EPI_WARPS 4
#endif
constexpr int kEpiWarps = TK_EPI_WARPS;
static_assert(kEpiWarps == 4 || kEpiWarps == 8, "TK_EPI_WARPS must be 4 or 8");
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kWorkerWarps = kThreads / 32;   // warps that run a stage's units; work items are cut for kThreads threads
// A kernel generated with stream warps is launched with kThreads + 32 * kStreamWarps threads: warps 6..9 do
// nothing but the stage's memory-bound pieces (gradient exchange, FP32 updates) while warps 0..5 run its GEMMs.
constexpr int kStreamWarps = 4;
constexpr int BM = 128;                // UMMA M
constexpr int BK = 64;                 // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
// The widest N tile any cta_group::1 GEMM of this kernel uses (a generated kernel defines it before
// including this file).  Narrower tiles take less room per K block, and the room goes into a deeper
// ring: a small GEMM is bound by the latency of its operand loads, so bytes in flight are what count.
#ifndef TK_RING_BN
#define TK_RING_BN 256
#endif
constexpr int kRingBN = TK_RING_BN;
static_assert(kRingBN == 64 || kRingBN == 128 || kRingBN == 256, "TK_RING_BN must be 64, 128 or 256");
// cta_group::1 ring: 4 x 48, 6 x 32 or 8 x 24 KiB; one slot less where eight epilogue warps need the room for
// their transposition buffers
constexpr int kStages = (kRingBN == 256 ? 4 : (kRingBN == 128 ? 6 : 8)) - (kEpiWarps == 8 ? 1 : 0);
constexpr int kStages2 = kEpiWarps == 8 ? 5 : 6;   // cta_group::2 ring: 6 x 32 KiB (5 with eight epilogue warps)
constexpr int kMaxStages = 8;
constexpr int kMaxBN = 256;            // accumulator pitch in TMEM columns
constexpr int kSlotA = BM * BK * 2;    // 16 KiB
constexpr int kSlotB = kRingBN * BK * 2;  // 8, 16 or 32 KiB
constexpr int kSlotBytes = kSlotA + kSlotB;
constexpr int kTmemCols = 512;         // two 256-column FP32 accumulators
constexpr int kDynSmem = 4 * (kSlotA + kMaxBN * BK * 2) + 1024;  // 192 KiB for any ring shape, +1024 for manual alignment
static_assert(kStages * kSlotBytes + 1024 <= kDynSmem && kStages <= kMaxStages, "ring does not fit");

// Stamp area (64-bit words) of kernels generated with stage stamps.
constexpr int kStampArrive = 64;       // + k: block 0 arrives at grid barrier k
constexpr int kStampLast = 128;        // + k: the last block arrives at grid barrier k
constexpr int kStampPeerWait = 192;    // + s: nanoseconds block 0 waited for peers' flags before stage s
constexpr int kStampTrace = 248;       // + point: role-level trace of one tile
constexpr uint32_t kTrustCarried = 1u; // launch flag: state untouched since the previous launch of this module
constexpr int kCarriedWord = 8;        // status word: values carried over from the previous launch are valid
constexpr int kCarryPhaseWord = 9;     // status word: which of the two copies of the carried values the next launch reads

enum : uint32_t {
    kOk = 0,
    kErrGridBarrier = 1,
    kErrSmemFull = 2,     // MMA issuer waited for TMA data
    kErrSmemEmpty = 3,    // producer waited for a free slot
    kErrTmemFull = 4,     // epilogue waited for the accumulator
    kErrTmemEmpty = 5,    // MMA issuer waited for the epilogue to drain
    kErrPeerFlag = 6,     // cross-GPU flag wait
};

// ----------------------------------------------------------------------------
// small PTX wrappers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t global_timer_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) { uint32_t v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_relaxed_gpu(uint32_t* p, uint32_t v) { asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) { uint32_t old; asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory"); return old; }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}

// Programmatic dependent launch.  A kernel launched with programmatic stream serialisation may start before
// its predecessor on the stream has finished: dependency_wait() returns once that predecessor has completed
// and its memory operations are visible (in an ordinary launch it returns at once), and
// launch_dependents() lets the NEXT kernel on the stream start its own prologue once every block of this
// one has got this far.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) { asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive FP32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (128-byte swizzle, sm_100 version bit set).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;     // descriptor version for sm_100
    d |= 2ull << 61;     // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16 with FP32 accumulation.  fmt: 0 = f16, 1 = bf16.  major: 0 = K, 1 = MN.
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int a_major, int b_major, int m, int n) {
    return (1u << 4) | (uint32_t(fmt) << 7) | (uint32_t(fmt) << 10) | (uint32_t(a_major) << 15) | (uint32_t(b_major) << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// ----------------------------------------------------------------------------
// per-CTA context
// ----------------------------------------------------------------------------
struct SharedState {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
    int bg_next;          // background pieces of this block taken from the front of the current stage's list
    int bg_back;          // ... and from its back
    int bg_taken;         // pieces handed out so far (front and back together)
    int bg_total;         // number of background pieces this block owns in the current stage
    int bg_count[8];      // per background unit of the stage: pieces this block owns
    int bg_first[8];      // ... and the first of its items that belongs to this block
    float reduce[32];
};

// Cross-GPU exchange state (see the exchange section below); unused by single-GPU kernels.
struct Dp {
    uint32_t* flags;      // this rank's header
    uint32_t epoch;       // epoch of the running launch
    uint32_t rank;
};

struct Ctx {
    Dp dp;
    uint32_t* sync;        // this launch's barrier word (phase bit + arrival count)
    uint32_t* status;      // {code, stage, block, detail}
    uint64_t* stamps;      // timestamp area when the kernel was generated with stage stamps, else null
    uint32_t flags;        // launch flags (kTrustCarried)
    uint64_t timeout_ns;
    uint32_t arrivals;     // blocks the grid barrier waits for (gridDim.x unless a test overrides it)
    SharedState* sh;
    uint8_t* slots;        // 1024-byte aligned pipeline slots
    float* epi;            // EpiStage: one 32 x 32 FP32 transpose buffer per epilogue warp
    uint32_t stage_id;
    // pipeline cursors; each role advances its own copy through the same tile sequence
    uint32_t slot, slot_phase;     // smem ring position and parity
    uint32_t acc, acc_phase;       // accumulator buffer and parity
    uint32_t tmem;
    int warp, lane;

    __device__ __forceinline__ bool aborted() const { return *reinterpret_cast<volatile uint32_t*>(&sh->abort) != 0; }
    __device__ __forceinline__ bool grid_aborted() const { return ld_relaxed_gpu(status) != 0; }
    __device__ __noinline__ void fail(uint32_t code, uint32_t detail) {
        if (atomicCAS(status, 0u, code) == 0u) {
            status[1] = stage_id;
            status[2] = blockIdx.x;
            status[3] = detail;
            __threadfence();
        }
        *reinterpret_cast<volatile uint32_t*>(&sh->abort) = 1u;
    }
    // Bounded mbarrier wait.  Returns false when the block is aborting.
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t code) {
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try(bar, parity)) return true;
        const uint64_t start = global_timer_ns();
        uint32_t polls = 0;
        while (!mbar_try(bar, parity)) {
            if (aborted()) return false;
            if ((++polls & 0x3F) == 0) {
                if (grid_aborted()) { *reinterpret_cast<volatile uint32_t*>(&sh->abort) = 1u; return false; }
                if (global_timer_ns() - start > timeout_ns) { fail(code, parity); return false; }
            }
        }
        return true;
    }
    __device__ __forceinline__ void advance_slot() { if (++slot == kStages) { slot = 0; slot_phase ^= 1; } }
    __device__ __forceinline__ void advance_slot2() { if (++slot == kStages2) { slot = 0; slot_phase ^= 1; } }
    __device__ __forceinline__ void advance_acc() { if (++acc == 2) { acc = 0; acc_phase ^= 1; } }
};

__device__ __forceinline__ void ctx_init(Ctx& c, uint32_t* sync, uint32_t* status, uint64_t timeout_ns, uint32_t arrivals, SharedState* sh, uint8_t* dyn, bool use_tc) {
    c.sync = sync; c.status = status; c.timeout_ns = timeout_ns; c.sh = sh;
    c.arrivals = arrivals ? arrivals : gridDim.x;
    c.slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~uintptr_t(1023));
    c.stage_id = 0; c.slot = 0; c.slot_phase = 0; c.acc = 0; c.acc_phase = 0; c.tmem = 0; c.epi = nullptr;
    c.stamps = nullptr; c.flags = 0;
    c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        sh->abort = 0;
        for (int i = 0; i < kStages; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->tmem_full[i], 1); mbar_init(&sh->tmem_empty[i], kEpiThreads / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (use_tc && c.warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (use_tc) c.tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);
}

__device__ __forceinline__ void ctx_finish(Ctx& c, bool use_tc) {
    tc_fence_before();
    __syncthreads();
    if (c.aborted()) {
        // Give TMA copies that nobody waited for time to land before shared memory is released.
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (use_tc && c.warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(c.tmem), "r"(kTmemCols) : "memory");
    }
}

// ----------------------------------------------------------------------------
// grid barrier: ONE word, one atomic per block and barrier, release/acquire at GPU scope.
// Bit 31 of the word is the barrier's phase, bits 0..30 count arrivals: block 0 adds
// 2^31 - (arrivals - 1), every other block adds 1, so the arrivals of one barrier add up to exactly
// 2^31: the phase bit flips when the last block arrives and the count is back at zero.  Nothing
// is reset and nothing is read before arriving, so the word serves any number of barriers,
// launches and CUDA-graph replays; a waiting block polls until the phase differs from the one its
// own atomic returned, and the last arriver recognises itself by the count it was handed.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void grid_barrier(Ctx& c) {
    fence_proxy_async();       // generic-proxy writes of this stage before later TMA reads
    __syncthreads();
    if (c.arrivals > 1 && threadIdx.x == 0 && !c.aborted()) {
        uint32_t* word = c.sync;
        if (c.stamps != nullptr && c.stage_id < 64) {
            // barrier stall evidence: when block 0 arrived, and when the last block did (the timer only
            // grows, so the maximum left by earlier launches never wins)
            const uint64_t now = global_timer_ns();
            if (blockIdx.x == 0) c.stamps[kStampArrive + c.stage_id] = now;
            atomicMax(reinterpret_cast<unsigned long long*>(c.stamps + kStampLast + c.stage_id), static_cast<unsigned long long>(now));
        }
        const bool leader = blockIdx.x == 0;
        const uint32_t before = atom_add_acq_rel_gpu(word, leader ? 0x80000000u - (c.arrivals - 1u) : 1u);
        const uint32_t counted = before & 0x7FFFFFFFu;
        const bool last = leader ? counted == c.arrivals - 1u : counted == 0x7FFFFFFFu;
        if (!last) {
            uint32_t polls = 0;
            uint64_t start = 0;
            while (((ld_acquire_gpu(word) ^ before) & 0x80000000u) == 0u) {
                if ((++polls & 0xFF) == 0) {
                    if (start == 0) start = global_timer_ns();
                    if (c.grid_aborted()) { *reinterpret_cast<volatile uint32_t*>(&c.sh->abort) = 1u; break; }
                    if (global_timer_ns() - start > c.timeout_ns) { c.fail(kErrGridBarrier, counted); break; }
                }
            }
        }
    }
    __syncthreads();
    fence_proxy_async();
    ++c.stage_id;
}

// Stage boundary of a kernel whose whole grid is ONE thread-block cluster: the hardware cluster
// barrier with release / acquire semantics at cluster scope (covers global memory), a fraction of
// the cost of a barrier through global memory.  It cannot time out, and it does not need to: every
// thread of every block reaches it, aborted or not, because an aborted block only skips work.
__device__ __forceinline__ void cluster_barrier(Ctx& c) {
    fence_proxy_async();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    fence_proxy_async();
    ++c.stage_id;
}

// ----------------------------------------------------------------------------
// rounding helpers: every IR value is rounded to its declared dtype
// ----------------------------------------------------------------------------
struct F32 { using T = float; static __device__ __forceinline__ float rnd(float x) { return x; } };
struct BF16 { using T = __nv_bfloat16; static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); } };
struct F16 { using T = __half; static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); } };

// Index dtypes (class labels and what one_hot derives from them) are carried as FP32 inside
// expressions; exact for magnitudes below 2^24.
struct I64 { using T = long long; static __device__ __forceinline__ float rnd(float x) { return x; } };
struct I32 { using T = int; static __device__ __forceinline__ float rnd(float x) { return x; } };
struct B8 { using T = bool; static __device__ __forceinline__ float rnd(float x) { return x != 0.0f ? 1.0f : 0.0f; } };
__device__ __forceinline__ float to_f32(long long x) { return static_cast<float>(x); }
__device__ __forceinline__ float to_f32(int x) { return static_cast<float>(x); }
__device__ __forceinline__ float to_f32(bool x) { return x ? 1.0f : 0.0f; }
__device__ __forceinline__ void from_f32(long long* p, float x) { *p = static_cast<long long>(x); }
__device__ __forceinline__ void from_f32(int* p, float x) { *p = static_cast<int>(x); }
__device__ __forceinline__ void from_f32(bool* p, float x) { *p = x != 0.0f; }
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ void from_f32(float* p, float x) { *p = x; }
__device__ __forceinline__ void from_f32(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
__device__ __forceinline__ void from_f32(__half* p, float x) { *p = __float2half_rn(x); }

__device__ __forceinline__ int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }
__device__ __forceinline__ int64_t imax(int64_t a, int64_t b) { return a > b ? a : b; }
// Pull `bytes` starting at p into L2 (one request per 128-byte line); used by epilogue warps to fetch the
// operands of the NEXT tile's epilogue while that tile's MMAs are still running.
__device__ __forceinline__ void prefetch_l2(const void* p, int bytes) {
    const char* q = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(p) & ~uintptr_t(127));
    const char* end = reinterpret_cast<const char*>(p) + bytes;
    for (; q < end; q += 128) asm volatile("prefetch.global.L2 [%0];" :: "l"(q));
}
__device__ __forceinline__ float relu(float x) { return x < 0.0f ? 0.0f : x; }   // keeps NaN like torch.relu

// W consecutive elements starting at p -> FP32.  Vector loads when p is 16-byte aligned and all W are valid.
template <int W>
__device__ __forceinline__ void ld_row(const float* p, int nvalid, float* out) {
    if constexpr (W % 4 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                const float4 v = *reinterpret_cast<const float4*>(p + j);
                out[j] = v.x; out[j + 1] = v.y; out[j + 2] = v.z; out[j + 3] = v.w;
            }
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j) out[j] = j < nvalid ? p[j] : 0.0f;
}
template <int W, typename T16>
__device__ __forceinline__ void ld_row16(const T16* p, int nvalid, float* out) {
    if constexpr (W % 8 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(p + j);
                const T16* h = reinterpret_cast<const T16*>(&raw);
#pragma unroll
                for (int e = 0; e < 8; ++e) out[j + e] = to_f32(h[e]);
            }
            return;
        }
    } else if constexpr (W % 4 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 7) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(p + j);
                const T16* h = reinterpret_cast<const T16*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) out[j + e] = to_f32(h[e]);
            }
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j) out[j] = j < nvalid ? to_f32(p[j]) : 0.0f;
}
template <int W> __device__ __forceinline__ void ld_row(const __nv_bfloat16* p, int nvalid, float* out) { ld_row16<W>(p, nvalid, out); }
template <int W> __device__ __forceinline__ void ld_row(const __half* p, int nvalid, float* out) { ld_row16<W>(p, nvalid, out); }

template <int W, typename TI>
__device__ __forceinline__ void ld_row_index(const TI* p, int nvalid, float* out) {
#pragma unroll
    for (int j = 0; j < W; ++j) out[j] = j < nvalid ? to_f32(p[j]) : 0.0f;
}
template <int W> __device__ __forceinline__ void ld_row(const long long* p, int nvalid, float* out) { ld_row_index<W>(p, nvalid, out); }
template <int W> __device__ __forceinline__ void ld_row(const int* p, int nvalid, float* out) { ld_row_index<W>(p, nvalid, out); }
template <int W> __device__ __forceinline__ void ld_row(const bool* p, int nvalid, float* out) { ld_row_index<W>(p, nvalid, out); }

// Strided variant: element j lives at p[j * step]; step 0 broadcasts one value.
template <int W, typename T>
__device__ __forceinline__ void ld_row_strided(const T* p, int64_t step, int nvalid, float* out) {
    if (step == 1) { ld_row<W>(p, nvalid, out); return; }
    if (step == 0) {
        const float v = to_f32(p[0]);
#pragma unroll
        for (int j = 0; j < W; ++j) out[j] = v;
        return;
    }
#pragma unroll
    for (int j = 0; j < W; ++j) out[j] = j < nvalid ? to_f32(p[j * step]) : 0.0f;
}

template <int W>
__device__ __forceinline__ void st_row(float* p, int nvalid, const float* v) {
    if constexpr (W % 4 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) *reinterpret_cast<float4*>(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j) if (j < nvalid) p[j] = v[j];
}
template <int W, typename T16>
__device__ __forceinline__ void st_row16(T16* p, int nvalid, const float* v) {
    if constexpr (W % 8 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 8) {
                uint4 raw;
                T16* h = reinterpret_cast<T16*>(&raw);
#pragma unroll
                for (int e = 0; e < 8; ++e) from_f32(h + e, v[j + e]);
                *reinterpret_cast<uint4*>(p + j) = raw;
            }
            return;
        }
    } else if constexpr (W % 4 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 7) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                uint2 raw;
                T16* h = reinterpret_cast<T16*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) from_f32(h + e, v[j + e]);
                *reinterpret_cast<uint2*>(p + j) = raw;
            }
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j) if (j < nvalid) from_f32(p + j, v[j]);
}
template <int W> __device__ __forceinline__ void st_row(__nv_bfloat16* p, int nvalid, const float* v) { st_row16<W>(p, nvalid, v); }
template <int W> __device__ __forceinline__ void st_row(__half* p, int nvalid, const float* v) { st_row16<W>(p, nvalid, v); }
template <int W, typename TI>
__device__ __forceinline__ void st_row_index(TI* p, int nvalid, const float* v) {
#pragma unroll
    for (int j = 0; j < W; ++j) if (j < nvalid) from_f32(p + j, v[j]);
}
template <int W> __device__ __forceinline__ void st_row(long long* p, int nvalid, const float* v) { st_row_index<W>(p, nvalid, v); }
template <int W> __device__ __forceinline__ void st_row(int* p, int nvalid, const float* v) { st_row_index<W>(p, nvalid, v); }
template <int W> __device__ __forceinline__ void st_row(bool* p, int nvalid, const float* v) { st_row_index<W>(p, nvalid, v); }

// Streaming variants for data touched exactly once by the kernel (FP32 masters read by the SGD
// expression, FP32 gradients and updated state written by it): the .cs policy marks the lines
// evict-first so they do not push GEMM operands out of L2.
__device__ __forceinline__ float4 ldg_stream(const float4* p) {
    float4 v;
    asm volatile("ld.global.cs.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void stg_stream(float4* p, float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
template <int W>
__device__ __forceinline__ void ld_row_stream(const float* p, int64_t step, int nvalid, float* out) {
    if constexpr (W % 4 == 0) {
        if (step == 1 && nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                const float4 v = ldg_stream(reinterpret_cast<const float4*>(p + j));
                out[j] = v.x; out[j + 1] = v.y; out[j + 2] = v.z; out[j + 3] = v.w;
            }
            return;
        }
    }
    ld_row_strided<W>(p, step, nvalid, out);
}
template <int W, typename T16>
__device__ __forceinline__ void ld_row_stream(const T16* p, int64_t step, int nvalid, float* out) { ld_row_strided<W>(p, step, nvalid, out); }
template <int W>
__device__ __forceinline__ void st_row_stream(float* p, int nvalid, const float* v) {
    if constexpr (W % 4 == 0) {
        if (nvalid >= W && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) stg_stream(reinterpret_cast<float4*>(p + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            return;
        }
    }
    st_row<W>(p, nvalid, v);
}
template <int W, typename T16>
__device__ __forceinline__ void st_row_stream(T16* p, int nvalid, const float* v) { st_row<W>(p, nvalid, v); }

// Row accesses of a tensor-core epilogue whose run of W elements is either wholly inside the tensor or wholly
// outside it (nvalid is 0 or W) and, when inside, starts on a 16-byte boundary (8 bytes for four 16-bit
// elements).  The code generator emits them where extents, strides and offsets prove both, and the host
// refuses a launch whose base pointers would break the proof; what they save is the element-wise fallback
// of ld_row / st_row, a third of an epilogue's instructions that never run but are fetched and stepped over
// in code that executes once per launch.  STREAM selects the evict-first forms for FP32 data touched once.
template <int W, bool STREAM>
__device__ __forceinline__ void ld_row_full(const float* p, int nvalid, float* out) {
    if constexpr (W % 4 == 0) {
        if (nvalid != 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                const float4 v = STREAM ? ldg_stream(reinterpret_cast<const float4*>(p + j)) : *reinterpret_cast<const float4*>(p + j);
                out[j] = v.x; out[j + 1] = v.y; out[j + 2] = v.z; out[j + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < W; ++j) out[j] = 0.0f;
        }
    } else {
        ld_row<W>(p, nvalid, out);
    }
}
template <int W, bool STREAM, typename T16>
__device__ __forceinline__ void ld_row_full(const T16* p, int nvalid, float* out) {
    static_assert(sizeof(T16) == 2, "16-bit element expected");
    if constexpr (W % 4 == 0) {
        if (nvalid != 0) {
            constexpr int V = W % 8 == 0 ? 8 : 4;
#pragma unroll
            for (int j = 0; j < W; j += V) {
                uint4 raw;
                if constexpr (V == 8) raw = *reinterpret_cast<const uint4*>(p + j);
                else { const uint2 half = *reinterpret_cast<const uint2*>(p + j); raw = make_uint4(half.x, half.y, 0u, 0u); }
                const T16* h = reinterpret_cast<const T16*>(&raw);
#pragma unroll
                for (int e = 0; e < V; ++e) out[j + e] = to_f32(h[e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < W; ++j) out[j] = 0.0f;
        }
    } else {
        ld_row<W>(p, nvalid, out);
    }
}
template <int W, bool STREAM>
__device__ __forceinline__ void st_row_full(float* p, int nvalid, const float* v) {
    if constexpr (W % 4 == 0) {
        if (nvalid != 0) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                if constexpr (STREAM) stg_stream(reinterpret_cast<float4*>(p + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
                else *reinterpret_cast<float4*>(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
    } else {
        st_row<W>(p, nvalid, v);
    }
}
template <int W, bool STREAM, typename T16>
__device__ __forceinline__ void st_row_full(T16* p, int nvalid, const float* v) {
    static_assert(sizeof(T16) == 2, "16-bit element expected");
    if constexpr (W % 4 == 0) {
        if (nvalid != 0) {
            constexpr int V = W % 8 == 0 ? 8 : 4;
#pragma unroll
            for (int j = 0; j < W; j += V) {
                uint4 raw;
                T16* h = reinterpret_cast<T16*>(&raw);
#pragma unroll
                for (int e = 0; e < V; ++e) from_f32(h + e, v[j + e]);
                if constexpr (V == 8) *reinterpret_cast<uint4*>(p + j) = raw;
                else *reinterpret_cast<uint2*>(p + j) = make_uint2(raw.x, raw.y);
            }
        }
    } else {
        st_row<W>(p, nvalid, v);
    }
}

// Barrier among the kThreads worker threads (warps 0..5) only: stream warps, where a kernel has them, are
// busy elsewhere and must not be waited for.  In a kernel of kThreads threads it is a block barrier.
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" :: "n"(kThreads) : "memory"); }

// FP32 sum over the worker threads; the total is valid in thread 0.  All kThreads worker threads must call it.
__device__ __forceinline__ float block_sum(Ctx& c, float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    worker_sync();
    if (c.lane == 0) c.sh->reduce[c.warp] = v;
    worker_sync();
    float total = 0.0f;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) total += c.sh->reduce[w];
    }
    return total;
}

// First work item of this block inside a unit whose items start at global position `base`
// of the stage's concatenated item list (items are dealt round-robin over blocks).
__device__ __forceinline__ int64_t first_item(int64_t base) {
    const int64_t g = gridDim.x;
    int64_t r = (static_cast<int64_t>(blockIdx.x) - base) % g;
    return r < 0 ? r + g : r;
}

// Tile rasterisation: groups of kGroupM tile rows are walked column by column so that the
// blocks of one wave share A rows and B columns in L2.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(int64_t t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int64_t per_group = static_cast<int64_t>(kGroupM) * tiles_n;
    const int group = static_cast<int>(t / per_group);
    const int first = group * kGroupM;
    const int rows = min(kGroupM, tiles_m - first);
    const int within = static_cast<int>(t - static_cast<int64_t>(group) * per_group);
    tm = first + within % rows;
    tn = within / rows;
}

// ----------------------------------------------------------------------------
// Cross-GPU exchange over peer-mapped ("symmetric") memory, one process per GPU.
//
// Every rank owns one symmetric buffer of identical layout: a 4 KiB header of 32-bit words followed
// by value regions.  Header: word 0 = number of launches completed (epoch), word 1 = this rank's
// index, words 16 + 64 * r + k = the epoch in which rank r last passed grid barrier k.  After a grid
// barrier that peers care about, threads 0 .. world-1 of one block each store the current epoch into
// that word of one rank's header with release semantics at system scope; everything the rank wrote
// before the barrier (to its own or to a peer's memory) is then visible to whoever acquires the
// word.  Waits are bounded like every other wait in this file.  In the scatter form peer memory is
// only ever WRITTEN (plain stores: contributions into the owner's staging area, means into every
// rank's result region); the multicast form reads and writes it through multimem instructions on
// the NVSwitch multicast mapping.  No TMA and no cluster-multicast load ever touches remote memory.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <typename T>
__device__ __forceinline__ T ld_volatile(const void* p) {
    T value;
    if constexpr (sizeof(T) == 2) {
        const unsigned short bits = *reinterpret_cast<const volatile unsigned short*>(p);
        memcpy(&value, &bits, 2);
    } else {
        const uint32_t bits = *reinterpret_cast<const volatile uint32_t*>(p);
        memcpy(&value, &bits, 4);
    }
    return value;
}

__device__ __forceinline__ void dp_init(Dp& d, void* symmetric_local) {
    d.flags = reinterpret_cast<uint32_t*>(symmetric_local);
    d.epoch = ld_relaxed_gpu(d.flags) + 1u;
    d.rank = ld_relaxed_gpu(d.flags + 1);
}
// Called by threads 0 .. world-1 of ONE block after grid barrier `barrier` (thread j tells rank j that this
// rank passed it): the release stores, each of which has to wait until this GPU's earlier writes are visible
// system-wide, then proceed side by side instead of one after the other.
__device__ __forceinline__ void dp_signal(const Dp& d, const void* const* peers, int peer, int barrier) {
    st_release_sys(reinterpret_cast<uint32_t*>(const_cast<void*>(peers[peer])) + 16 + d.rank * 64 + barrier, d.epoch);
}
// Called by all threads of a block: returns once every rank has passed grid barrier `barrier` of this epoch.
// Thread j watches rank j's flag, so the (system-scope) polls of the ranks overlap.
__device__ __forceinline__ void dp_wait(Ctx& c, const Dp& d, int world, int barrier) {
    const bool stamped = c.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && c.stage_id < 56;
    const uint64_t begun = stamped ? global_timer_ns() : 0;
    if (threadIdx.x < world && !c.aborted()) {
        const int j = threadIdx.x;
        const uint32_t* word = d.flags + 16 + j * 64 + barrier;
        uint32_t polls = 0;
        uint64_t start = 0;
        while (static_cast<int32_t>(ld_acquire_sys(word) - d.epoch) < 0) {
            if ((++polls & 0x3F) == 0) {
                if (start == 0) start = global_timer_ns();
                if (c.grid_aborted() || c.aborted()) { *reinterpret_cast<volatile uint32_t*>(&c.sh->abort) = 1u; break; }
                if (global_timer_ns() - start > c.timeout_ns) { c.fail(kErrPeerFlag, static_cast<uint32_t>(j * 64 + barrier)); break; }
            }
        }
    }
    __syncthreads();
    if (stamped) c.stamps[kStampPeerWait + c.stage_id] = global_timer_ns() - begun;
}
__device__ __forceinline__ void dp_finish(const Dp& d) { st_relaxed_gpu(d.flags, d.epoch); }

// Store `nvalid` of W consecutive elements of a value that is about to be averaged across ranks, starting at
// flat element index e, into the staging area of the rank that owns their chunk: chunk c = e / (THREADS * VEC)
// belongs to rank c % WORLD and is staged there at [this rank][c / WORLD].  Producers (GEMM epilogues,
// reduction finishes) call this instead of a local store, so the contribution crosses NVLink as posted
// writes while the producing stage runs and nobody ever reads remote memory.
template <int W, int WORLD, typename T>
__device__ __forceinline__ void st_row_scatter(const void* const* peers, uint64_t region_offset, uint64_t owned_bytes,
                                               uint32_t rank, int64_t e, int nvalid, const float* v) {
    constexpr int64_t chunk = static_cast<int64_t>(kThreads) * (16 / static_cast<int>(sizeof(T)));
    if (nvalid <= 0) return;
    if ((e % W) == 0 && (chunk % W) == 0) {                    // the run lies inside one chunk
        const int64_t c = e / chunk;
        char* base = reinterpret_cast<char*>(const_cast<void*>(peers[c % WORLD])) + region_offset + rank * owned_bytes;
        st_row<W>(reinterpret_cast<T*>(base) + (c / WORLD) * chunk + e % chunk, nvalid, v);
        return;
    }
    for (int j = 0; j < W && j < nvalid; ++j) {
        const int64_t c = (e + j) / chunk;
        char* base = reinterpret_cast<char*>(const_cast<void*>(peers[c % WORLD])) + region_offset + rank * owned_bytes;
        from_f32(reinterpret_cast<T*>(base) + (c / WORLD) * chunk + (e + j) % chunk, v[j]);
    }
}

// Owned chunks one exchange work item covers = 16-byte loads each thread keeps in flight through the switch.
// A generated kernel defines TK_EXCHANGE_CHUNKS to what its planner cut the items for.
#ifndef TK_EXCHANGE_CHUNKS
#define TK_EXCHANGE_CHUNKS 8
#endif
constexpr int kExchangeChunksPerItem = TK_EXCHANGE_CHUNKS;

// Mean over ranks of a dense value, rounded to T: chunk c (THREADS x 16 bytes) is reduced by rank
// c % WORLD, which reads every rank's contribution from its own staging area (filled by
// st_row_scatter; fixed order, FP32 sum), scales by 1/WORLD, rounds, and stores the result into
// every rank's result region.  Every rank ends up with the bit-identical mean.  One item = kExchangeChunksPerItem owned chunks.
template <typename R, int WORLD>
__device__ __noinline__ void exchange_mean_item(const Dp& d, const void* const* peers, uint64_t src_offset, uint64_t owned_bytes,
                                                   uint64_t dst_offset, int64_t numel, int64_t it, int tid) {
    using T = typename R::T;
    constexpr int VEC = 16 / static_cast<int>(sizeof(T));
    const int64_t chunk = static_cast<int64_t>(kThreads) * VEC;
    const int64_t chunks = (numel + chunk - 1) / chunk;
    const float scale = 1.0f / static_cast<float>(WORLD);
    // G chunks are pulled together so that G * WORLD 128-bit loads per thread are in flight: a remote
    // load takes a few microseconds, and NVLink only fills up with megabytes outstanding per GPU.
    constexpr int G = WORLD <= 2 ? 8 : (WORLD <= 4 ? 4 : 2);
    // every rank's contribution to the chunks this rank owns has been staged in LOCAL memory by its producer
    const char* staging = reinterpret_cast<const char*>(peers[d.rank]) + src_offset;
    {
#pragma unroll 1
        for (int u0 = 0; u0 < kExchangeChunksPerItem; u0 += G) {
            uint4 raw[G][WORLD];
            int64_t e0[G];
            const char* staged[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const int64_t slot = it * kExchangeChunksPerItem + u0 + g;           // this rank's slot-th owned chunk
                const int64_t owned = slot * WORLD + d.rank;
                e0[g] = owned < chunks ? owned * chunk + static_cast<int64_t>(tid) * VEC : numel;
                staged[g] = staging + (slot * chunk + static_cast<int64_t>(tid) * VEC) * sizeof(T);
                if (e0[g] + VEC <= numel) {
#pragma unroll
                    for (int j = 0; j < WORLD; ++j) raw[g][j] = ld_relaxed_sys_v4(staged[g] + j * owned_bytes);
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (e0[g] >= numel) continue;
                const uint64_t byte = static_cast<uint64_t>(e0[g]) * sizeof(T);
                if (e0[g] + VEC <= numel) {
                    float sum[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) sum[e] = 0.0f;
#pragma unroll
                    for (int j = 0; j < WORLD; ++j) {
                        const T* part = reinterpret_cast<const T*>(&raw[g][j]);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) sum[e] += to_f32(part[e]);
                    }
                    uint4 packed;
                    T* out = reinterpret_cast<T*>(&packed);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) from_f32(out + e, sum[e] * scale);
#pragma unroll
                    for (int j = 0; j < WORLD; ++j) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(const_cast<void*>(peers[j])) + dst_offset + byte) = packed;
                } else {
                    for (int64_t e = e0[g]; e < numel; ++e) {
                        float sum = 0.0f;
                        for (int j = 0; j < WORLD; ++j)
                            sum += to_f32(ld_volatile<T>(staged[g] + j * owned_bytes + (e - e0[g]) * sizeof(T)));
                        T value;
                        from_f32(&value, sum * scale);
                        for (int j = 0; j < WORLD; ++j)
                            *reinterpret_cast<T*>(reinterpret_cast<char*>(const_cast<void*>(peers[j])) + dst_offset + e * sizeof(T)) = value;
                    }
                }
            }
        }
    }
}

template <typename R, int WORLD>
__device__ __forceinline__ void exchange_mean(Ctx& c, const void* const* peers, uint64_t src_offset, uint64_t owned_bytes,
                                              uint64_t dst_offset, int64_t numel, int64_t item_base, int64_t items) {
    for (int64_t it = first_item(item_base); it < items && !c.aborted(); it += gridDim.x)
        exchange_mean_item<R, WORLD>(c.dp, peers, src_offset, owned_bytes, dst_offset, numel, it, threadIdx.x);
}

// The same exchange through the NVSwitch multicast mapping of the symmetric buffer (`mc` is this
// rank's pointer to it).  Every rank keeps its contribution in its OWN buffer; the owner of a chunk
// issues one multimem.ld_reduce per 16 bytes, which the switch answers with the FP32-accumulated sum
// over all ranks (so a chunk crosses this rank's links once, already reduced), scales and rounds
// it, and one multimem.st delivers the mean to every rank's result region.  Per rank and direction
// this moves (WORLD - 1) / WORLD + 1 / WORLD of the value instead of 2 (WORLD - 1) / WORLD.
// The sum comes back rounded to T; scaling by 1 / WORLD afterwards is exact for power-of-two WORLD.
// Elements of a last, partial 16-byte group go over the unicast peer pointers.
template <typename T>
__device__ __forceinline__ uint4 multimem_sum_v4(const void* p) {
    uint4 v;
    if constexpr (sizeof(T) == 4)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else if constexpr (std::is_same<T, __nv_bfloat16>::value)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st_v4(void* p, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename R, int WORLD>
__device__ __noinline__ void exchange_mean_mc_item(const Dp& d, const void* const* peers, const void* mc, uint64_t src_offset,
                                                      uint64_t dst_offset, int64_t numel, int64_t it, int tid) {
    using T = typename R::T;
    static_assert(std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value,
                  "exchanged values are floating point");
    constexpr int VEC = 16 / static_cast<int>(sizeof(T));
    constexpr int G = kExchangeChunksPerItem;
    const int64_t chunk = static_cast<int64_t>(kThreads) * VEC;
    const int64_t chunks = (numel + chunk - 1) / chunk;
    const float scale = 1.0f / static_cast<float>(WORLD);
    char* base = reinterpret_cast<char*>(const_cast<void*>(mc));
    // This thread's 16 bytes of the item's g-th chunk sit a compile-time stride behind those of chunk 0, so
    // one 64-bit address and immediates serve all G loads and stores (G 64-bit indices next to G loaded
    // vectors would not fit the register budget).
    constexpr int64_t kStride = static_cast<int64_t>(WORLD) * kThreads * VEC;          // elements between owned chunks
    const int64_t e_first = ((it * G) * WORLD + d.rank) * chunk + static_cast<int64_t>(tid) * VEC;
    const char* src = base + src_offset + static_cast<uint64_t>(e_first) * sizeof(T);
    char* dst = base + dst_offset + static_cast<uint64_t>(e_first) * sizeof(T);
    uint4 raw[G];
#pragma unroll
    for (int g = 0; g < G; ++g)
        if (e_first + g * kStride + VEC <= numel) raw[g] = multimem_sum_v4<T>(src + g * kStride * static_cast<int64_t>(sizeof(T)));
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int64_t e0 = e_first + g * kStride;
        if (e0 >= numel) continue;
        if (e0 + VEC <= numel) {
            const T* part = reinterpret_cast<const T*>(&raw[g]);
            uint4 packed;
            T* out = reinterpret_cast<T*>(&packed);
#pragma unroll
            for (int e = 0; e < VEC; ++e) from_f32(out + e, to_f32(part[e]) * scale);
            multimem_st_v4(dst + g * kStride * static_cast<int64_t>(sizeof(T)), packed);
        } else {
            for (int64_t e = e0; e < numel; ++e) {
                float sum = 0.0f;
                for (int j = 0; j < WORLD; ++j)
                    sum += to_f32(ld_volatile<T>(reinterpret_cast<const char*>(peers[j]) + src_offset + e * sizeof(T)));
                T value;
                from_f32(&value, sum * scale);
                for (int j = 0; j < WORLD; ++j)
                    *reinterpret_cast<T*>(reinterpret_cast<char*>(const_cast<void*>(peers[j])) + dst_offset + e * sizeof(T)) = value;
            }
        }
    }
}

template <typename R, int WORLD>
__device__ __forceinline__ void exchange_mean_mc(Ctx& c, const void* const* peers, const void* mc, uint64_t src_offset,
                                                 uint64_t dst_offset, int64_t numel, int64_t item_base, int64_t items) {
    for (int64_t it = first_item(item_base); it < items && !c.aborted(); it += gridDim.x)
        exchange_mean_mc_item<R, WORLD>(c.dp, peers, mc, src_offset, dst_offset, numel, it, threadIdx.x);
}

// ----------------------------------------------------------------------------
// Background work.  Memory-bound units of a stage (flat pointwise streams, exchange units) are cut
// into per-warp pieces that the block's STREAM WARPS (warps 6..9 of a kernel generated with them)
// execute while warps 0..5 run the stage's GEMM tiles, so HBM and NVLink traffic overlaps the MMAs
// of the same stage on every SM.  A stage's functor Bg maps an ordinal of this block to (unit,
// item, 32-thread slice); ordinals are handed out with a shared-memory counter, and whatever is
// left when the GEMM tiles are done is drained by all warps.
// ----------------------------------------------------------------------------
struct NoBg {
    static constexpr bool kActive = false;
    template <typename Params> static __device__ __forceinline__ void run(const Params&, Ctx&, int, int) {}
};

// The list is worked from both ends: the pieces at the front are the HBM-bound streams, the ones at the back
// the exchanges that are bound by NVLink, and warps coming from either side keep both busy at once.
template <typename Bg, typename Params>
__device__ __forceinline__ bool bg_step(Ctx& c, const Params& P, bool from_back) {
    int ordinal = -1;
    if (c.lane == 0 && !c.aborted()) {              // one lane decides for the warp
        const int total = *reinterpret_cast<volatile int*>(&c.sh->bg_total);
        if (atomicAdd(&c.sh->bg_taken, 1) < total)
            ordinal = from_back ? total - 1 - atomicAdd(&c.sh->bg_back, 1) : atomicAdd(&c.sh->bg_next, 1);
    }
    ordinal = __shfl_sync(0xffffffffu, ordinal, 0);
    if (ordinal < 0) return false;
    Bg::run(P, c, ordinal, c.lane);
    return true;
}
template <typename Bg, typename Params>
__device__ __forceinline__ void bg_drain(Ctx& c, const Params& P) {
    if constexpr (Bg::kActive) {
        __syncwarp();
        const bool from_back = c.warp >= kWorkerWarps + kStreamWarps / 2;
        while (bg_step<Bg>(c, P, from_back)) {}
    }
}
// Number of items of a unit (n items starting at list position `base`) that this block owns.
__device__ __forceinline__ int64_t owned_items(int64_t base, int64_t n) {
    const int64_t first = first_item(base);
    return first < n ? (n - first + gridDim.x - 1) / gridDim.x : 0;
}

// ----------------------------------------------------------------------------
// Epilogue chunk.  tcgen05.ld hands every lane one accumulator ROW (32 consecutive columns), so a
// warp-wide global access would touch 32 different rows.  The chunk is therefore transposed through
// a padded shared-memory buffer: afterwards 8 (or 4) lanes share a row and each warp-wide 128-bit
// access covers whole 128-byte (or 64-byte) row segments.  All rows' loads are issued before the
// first store (Epi::run_rows).
// ----------------------------------------------------------------------------
constexpr int kEpiPitch = 36;                       // floats per staged row: 16-byte aligned, conflict-free
struct alignas(16) EpiStage { float t[kEpiThreads / 32][32][kEpiPitch]; };

// Operands of one chunk in the layout the warp will consume them in (see epilogue_chunk).
template <typename Epi>
struct EpiOps {
    using type = typename std::conditional<Epi::kWide, typename Epi::template Ops<8, 4>, typename Epi::template Ops<4, 8>>::type;
};

// Issue the global loads of the chunk at (row0, col0): called one chunk ahead of epilogue_chunk, so that the
// loads are in flight while the previous chunk's accumulator is read, transposed, combined and stored.
template <typename Epi, typename Params>
__device__ __forceinline__ void epilogue_fetch(Ctx& c, const Params& P, int row0, int col0, int ncols, typename EpiOps<Epi>::type& L) {
    if constexpr (Epi::kWide) {
        const int cq = (c.lane & 7) * 4, rq = c.lane >> 3;
        Epi::template load_rows<8, 4>(P, row0 + rq, 4, col0 + cq, max(0, min(4, ncols - cq)), L);
    } else {
        const int cq = (c.lane & 3) * 8, rq = c.lane >> 2;
        Epi::template load_rows<4, 8>(P, row0 + rq, 8, col0 + cq, max(0, min(8, ncols - cq)), L);
    }
}

template <typename Epi, typename Params>
__device__ __forceinline__ void epilogue_chunk(Ctx& c, const Params& P, const float* acc, int row0, int col0, int ncols,
                                               const typename EpiOps<Epi>::type& L) {
    float* stage = c.epi + (c.warp - 2) * 32 * kEpiPitch;
    float* mine = stage + c.lane * kEpiPitch;
#pragma unroll
    for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(mine + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    __syncwarp();
    if constexpr (Epi::kWide) {
        const int cq = (c.lane & 7) * 4, rq = c.lane >> 3;      // runs of 4 columns, rows rq, rq+4, ...
        float v[8][4];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float4 q = *reinterpret_cast<const float4*>(stage + (rq + 4 * r) * kEpiPitch + cq);
            v[r][0] = q.x; v[r][1] = q.y; v[r][2] = q.z; v[r][3] = q.w;
        }
        Epi::template run_rows<8, 4>(P, row0 + rq, 4, col0 + cq, max(0, min(4, ncols - cq)), v, L);
    } else {
        const int cq = (c.lane & 3) * 8, rq = c.lane >> 2;      // runs of 8 columns, rows rq, rq+8, ...
        float v[4][8];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float4 q0 = *reinterpret_cast<const float4*>(stage + (rq + 8 * r) * kEpiPitch + cq);
            const float4 q1 = *reinterpret_cast<const float4*>(stage + (rq + 8 * r) * kEpiPitch + cq + 4);
            v[r][0] = q0.x; v[r][1] = q0.y; v[r][2] = q0.z; v[r][3] = q0.w;
            v[r][4] = q1.x; v[r][5] = q1.y; v[r][6] = q1.z; v[r][7] = q1.w;
        }
        Epi::template run_rows<4, 8>(P, row0 + rq, 8, col0 + cq, max(0, min(8, ncols - cq)), v, L);
    }
    __syncwarp();
}

// The epilogue of one accumulator tile of TN columns starting at tile column `tile_col0`, as seen by one warp:
// the 32-column chunks `chunk0`, `chunk0 + step`, ... (step 1: the warp has its TMEM quarter to itself; step 2:
// two warps share the quarter and take alternate chunks).  With Epi::kPipelined the operands of the warp's
// next chunk are requested before the current one is read out of TMEM (two chunks per iteration, so that the
// two operand buffers alternate without run-time indexing); `first` must then already hold those of chunk
// `chunk0`, as it must with Epi::kFetchFirst (the caller requested them before it waited for the
// accumulator; later chunks fetch their own at their start).
template <int TN, typename Epi, typename Params>
__device__ __forceinline__ void epilogue_tile(Ctx& c, const Params& P, uint32_t taddr, int row0, int tile_col0, int N,
                                              typename EpiOps<Epi>::type& first, int chunk0 = 0, int step = 1) {
    const int stride = 32 * step;                          // columns between this warp's consecutive chunks
    if constexpr (!Epi::kPipelined) {
        // one chunk body, executed once per chunk: half the code of the look-ahead form below, which matters in
        // kernels whose every GEMM runs its epilogue a handful of times per launch (instruction fetch is cold)
#pragma unroll 1
        for (int cc = 32 * chunk0; cc < TN; cc += stride) {
            const int col0 = tile_col0 + cc;
            if (col0 >= N) break;                          // warp-uniform
            if (!(Epi::kFetchFirst && cc == 32 * chunk0)) epilogue_fetch<Epi>(c, P, row0, col0, min(32, N - col0), first);
            float acc[32];
            tc_ld32(taddr + cc, acc);
            tc_wait_ld();
            epilogue_chunk<Epi>(c, P, acc, row0, col0, min(32, N - col0), first);
        }
        return;
    }
    typename EpiOps<Epi>::type second;
#pragma unroll 1
    for (int cc = 32 * chunk0; cc < TN; cc += 2 * stride) {
        const int col0 = tile_col0 + cc;
        if (col0 >= N) break;                              // warp-uniform
        const bool pair = cc + stride < TN && col0 + stride < N;
        if (pair) epilogue_fetch<Epi>(c, P, row0, col0 + stride, min(32, N - col0 - stride), second);
        float acc[32];
        tc_ld32(taddr + cc, acc);
        tc_wait_ld();
        epilogue_chunk<Epi>(c, P, acc, row0, col0, min(32, N - col0), first);
        if (!pair) break;
        if (cc + 2 * stride < TN && col0 + 2 * stride < N) epilogue_fetch<Epi>(c, P, row0, col0 + 2 * stride, min(32, N - col0 - 2 * stride), first);
        tc_ld32(taddr + cc + stride, acc);
        tc_wait_ld();
        epilogue_chunk<Epi>(c, P, acc, row0, col0 + stride, min(32, N - col0 - stride), second);
    }
}

// ----------------------------------------------------------------------------
// tcgen05 GEMM unit.  C[M,N] = A[M,K] * B[K,N], 16-bit operands, FP32 accumulate in TMEM.
//   A_MN / B_MN: operand is MN-major in global memory (unit stride along M resp. N)
//                instead of K-major (unit stride along K).
//   Epi::run<32>(P, row, col0, nvalid, acc) consumes 32 accumulator columns of one row.
// Tensor maps: K-major operands use a {64 (K), rows} box; MN-major operands use a
// {64 (MN), 64 (K)} box issued once per 64-wide MN atom.  Out-of-range parts of a box are
// zero-filled by TMA, which is what makes M, N and K tails work.
// ----------------------------------------------------------------------------
// Optional role-level timestamps of ONE stage's first tensor-core tile (compile with
// -DTK_TRACE_STAGE=<stage>): the thread that reaches point k while working on tile 0 of that stage
// writes the global timer to stamp slot kStampTrace + k.  Points: 0 producer starts, 1 last TMA issued,
// 2 first operands landed, 3 last MMA committed, 4 accumulator seen complete, 5 epilogue done.
#ifdef TK_TRACE_STAGE
#define TK_TRACE(point, tile) do { if (c.stage_id == TK_TRACE_STAGE && (tile) == 0) P.stamps[tk::kStampTrace + (point)] = global_timer_ns(); } while (0)
#else
#define TK_TRACE(point, tile) do { } while (0)
#endif

template <int BN, bool A_MN, bool B_MN, int FMT, typename Epi, typename Bg, typename Params>
__device__ __forceinline__ void gemm_tc(Ctx& c, const Params& P, const CUtensorMap* map_a, const CUtensorMap* map_b,
                                        int M, int N, int K, int64_t item_base) {
    static_assert(BN % 64 == 0 && BN <= kRingBN, "BN must be a multiple of 64 within the ring's tile width");
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n;
    const int kblocks = (K + BK - 1) / BK;
    const int64_t step = gridDim.x;
    constexpr uint32_t kBytes = BM * BK * 2 + BN * BK * 2;
    SharedState* sh = c.sh;

    if (c.warp == 0) {
        if (c.lane == 0) {
            for (int64_t t = first_item(item_base); t < tiles && !c.aborted(); t += step) {
                int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
                TK_TRACE(0, t);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!c.wait(&sh->empty[c.slot], c.slot_phase ^ 1, kErrSmemEmpty)) break;
                    uint8_t* sa = c.slots + c.slot * kSlotBytes;
                    uint8_t* sb = sa + kSlotA;
                    mbar_expect_tx(&sh->full[c.slot], kBytes);
                    if constexpr (A_MN) {
#pragma unroll
                        for (int a = 0; a < BM / 64; ++a) tma_load_2d(sa + a * 8192, map_a, &sh->full[c.slot], tm * BM + a * 64, kb * BK);
                    } else {
                        tma_load_2d(sa, map_a, &sh->full[c.slot], kb * BK, tm * BM);
                    }
                    if constexpr (B_MN) {
#pragma unroll
                        for (int b = 0; b < BN / 64; ++b) tma_load_2d(sb + b * 8192, map_b, &sh->full[c.slot], tn * BN + b * 64, kb * BK);
                    } else {
                        tma_load_2d(sb, map_b, &sh->full[c.slot], kb * BK, tn * BN);
                    }
                    c.advance_slot();
                }
                TK_TRACE(1, t);
            }
        }
        __syncwarp();
    } else if (c.warp == 1) {
        if (c.lane == 0) {
            constexpr uint32_t idesc = umma_idesc(FMT, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
            for (int64_t t = first_item(item_base); t < tiles && !c.aborted(); t += step) {
                if (!c.wait(&sh->tmem_empty[c.acc], c.acc_phase ^ 1, kErrTmemEmpty)) break;
                tc_fence_after();
                const uint32_t d_tmem = c.tmem + c.acc * kMaxBN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!c.wait(&sh->full[c.slot], c.slot_phase, kErrSmemFull)) { ok = false; break; }
                    tc_fence_after();
                    if (kb == 0) TK_TRACE(2, t);
                    const uint32_t sa = smem_u32(c.slots + c.slot * kSlotBytes);
                    const uint32_t sb = sa + kSlotA;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = A_MN ? umma_desc(sa + k * 2048, 8192, 1024) : umma_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? umma_desc(sb + k * 2048, 8192, 1024) : umma_desc(sb + k * 32, 16, 1024);
                        tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(&sh->empty[c.slot]);     // frees the slot once these MMAs have read it
                    c.advance_slot();
                }
                if (!ok) break;
                tc_commit(&sh->tmem_full[c.acc]);      // accumulator complete
                TK_TRACE(3, t);
                c.advance_acc();
            }
        }
        __syncwarp();
    } else if (c.warp < 2 + kEpiWarps) {
        const int quarter = c.warp & 3;                // TMEM lanes this warp may read
        const int chunk0 = (c.warp - 2) >> 2;          // wide epilogue: warps 6..9 start one chunk later ...
        constexpr int kChunkStep = kEpiWarps / 4;      // ... and every warp takes every other chunk
        for (int64_t t = first_item(item_base); t < tiles && !c.aborted(); t += step) {
            int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
            if (chunk0 == 0 && t == first_item(item_base)) {
                // the block's first tile of this unit: nobody fetched its epilogue operands yet, and these warps
                // are idle until the accumulator is complete
                const int prow = tm * BM + quarter * 32 + c.lane;
                if (prow < M) Epi::prefetch(P, prow, tn * BN, min(BN, N - tn * BN));
            }
            if (chunk0 == 0 && t + step < tiles) {
                int pm, pn; tile_coords(t + step, tiles_m, tiles_n, pm, pn);
                const int prow = pm * BM + quarter * 32 + c.lane;
                if (prow < M && pn * BN < N) Epi::prefetch(P, prow, pn * BN, min(BN, N - pn * BN));
            }
            const int row0 = tm * BM + quarter * 32;
            typename EpiOps<Epi>::type operands;
            if constexpr (Epi::kPipelined || Epi::kFetchFirst) {               // in flight during the wait
                if (tn * BN + 32 * chunk0 < N) epilogue_fetch<Epi>(c, P, row0, tn * BN + 32 * chunk0, min(32, N - tn * BN - 32 * chunk0), operands);
            }
            if (!c.wait(&sh->tmem_full[c.acc], c.acc_phase, kErrTmemFull)) break;
            tc_fence_after();
            if (threadIdx.x == 64) TK_TRACE(4, t);
            const uint32_t taddr = c.tmem + c.acc * kMaxBN + (static_cast<uint32_t>(quarter * 32) << 16);
            epilogue_tile<BN, Epi>(c, P, taddr, row0, tn * BN, N, operands, chunk0, kChunkStep);
            tc_fence_before();
            __syncwarp();
            if (c.lane == 0) mbar_arrive(&sh->tmem_empty[c.acc]);
            if (threadIdx.x == 64) TK_TRACE(5, t);
            c.advance_acc();
        }
    }
}

// ----------------------------------------------------------------------------
// SIMT GEMM unit (exact FP32 accumulation with fmaf, sequential in K per output).
// Operands are read through arbitrary element strides and converted to FP32, optionally
// re-rounded to a 16-bit type first (a cast folded into the load).  32x32 output tile per
// block-iteration, 128 compute threads each owning a 2x4 strip.  The staging buffers live at the
// start of the dynamic shared memory (idle whenever all threads of a block are inside this unit).
// ----------------------------------------------------------------------------
constexpr int kSimtK = 128;            // K depth staged per step: few steps, many loads in flight per step
struct alignas(16) SimtSmem { float a[32][kSimtK + 1]; float pad[4 - (32 * (kSimtK + 1)) % 4]; float b[kSimtK][36]; };

template <int KS, typename TA, typename RA, typename TB, typename RB, typename Epi, typename Params>
__device__ __forceinline__ void gemm_simt(Ctx& c, const Params& P, SimtSmem* sm, const TA* A, int64_t a_rs, int64_t a_ks,
                                          const TB* B, int64_t b_ks, int64_t b_cs, int M, int N, int K, int64_t item_base) {
    // KS: the K depth staged per step (32, 64 or 128 = kSimtK, the buffers' size).  The loads of a step are
    // unrolled per staged position, so a product whose K is 32 should not carry the code of 128.
    static_assert(KS == 32 || KS == 64 || KS == kSimtK, "staging depth");
    const int tiles_n = (N + 31) / 32;
    const int64_t tiles = static_cast<int64_t>((M + 31) / 32) * tiles_n;
    const int tid = threadIdx.x;
    const int ty = tid / 8, tx = tid % 8;      // valid for tid < 128: rows 2*ty.., cols 4*tx..
    const bool a_k_fast = a_ks <= a_rs, b_n_fast = b_cs <= b_ks;
    for (int64_t t = first_item(item_base); t < tiles; t += gridDim.x) {
        const int row0 = static_cast<int>(t / tiles_n) * 32, col0 = static_cast<int>(t % tiles_n) * 32;
        float acc[2][4] = {};
        for (int k0 = 0; k0 < K; k0 += KS) {
            const int depth = min(KS, K - k0);
            worker_sync();
            // Stage A[32, depth] and B[depth, 32].  Positions are decomposed against the fixed staging
            // depth (shifts and masks, no division by a runtime value) and the part beyond `depth` is
            // skipped.  A thread issues ALL of its loads of the step (22 per operand) before its first
            // shared-memory store: one round trip to memory per step.  Consecutive threads walk the
            // unit-stride axis of each operand.
            constexpr int kPerThread = (32 * KS + kThreads - 1) / kThreads;
            float va[kPerThread], vb[kPerThread];
#pragma unroll
            for (int u = 0; u < kPerThread; ++u) {
                const int p = tid + u * kThreads;
                const int ar = a_k_fast ? p / KS : p % 32, ak = a_k_fast ? p % KS : p / 32;
                const int bk = b_n_fast ? p / 32 : p % KS, bc = b_n_fast ? p % 32 : p / KS;
                const bool in_tile = p < 32 * KS;
                const int gr = row0 + ar, gc = col0 + bc;
                va[u] = (in_tile && ak < depth && gr < M) ? RA::rnd(to_f32(A[static_cast<int64_t>(gr) * a_rs + static_cast<int64_t>(k0 + ak) * a_ks])) : 0.0f;
                vb[u] = (in_tile && bk < depth && gc < N) ? RB::rnd(to_f32(B[static_cast<int64_t>(k0 + bk) * b_ks + static_cast<int64_t>(gc) * b_cs])) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kPerThread; ++u) {
                const int p = tid + u * kThreads;
                const int ar = a_k_fast ? p / KS : p % 32, ak = a_k_fast ? p % KS : p / 32;
                const int bk = b_n_fast ? p / 32 : p % KS, bc = b_n_fast ? p % 32 : p / KS;
                if (p < 32 * KS) {
                    if (ak < depth) sm->a[ar][ak] = va[u];
                    if (bk < depth) sm->b[bk][bc] = vb[u];
                }
            }
            worker_sync();
            if (tid < 128) {
#pragma unroll 8
                for (int k = 0; k < depth; ++k) {
                    const float a0 = sm->a[2 * ty][k], a1 = sm->a[2 * ty + 1][k];
                    const float4 b = *reinterpret_cast<const float4*>(&sm->b[k][4 * tx]);
                    acc[0][0] = fmaf(a0, b.x, acc[0][0]); acc[0][1] = fmaf(a0, b.y, acc[0][1]);
                    acc[0][2] = fmaf(a0, b.z, acc[0][2]); acc[0][3] = fmaf(a0, b.w, acc[0][3]);
                    acc[1][0] = fmaf(a1, b.x, acc[1][0]); acc[1][1] = fmaf(a1, b.y, acc[1][1]);
                    acc[1][2] = fmaf(a1, b.z, acc[1][2]); acc[1][3] = fmaf(a1, b.w, acc[1][3]);
                }
            }
        }
        if (tid < 128) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = row0 + 2 * ty + i, cc = col0 + 4 * tx;
                if (r < M && cc < N) Epi::template run<4>(P, r, cc, min(4, N - cc), acc[i]);
            }
        }
    }
}

// ----------------------------------------------------------------------------
// GEMV unit (M == 1): y[n] = sum_k a[k] * B[k, n], FP32 accumulation.  Operands may be
// stored in a wider type and rounded on load (RA / RB), which folds an FP32 -> BF16 cast of a
// master weight into the read.  128-bit loads, warp-shuffle reductions.
//   B_KMAJOR: B has unit stride along K (a transposed weight view): one warp per output
//             column, each lane takes 8 consecutive K elements per step.
//   otherwise B has unit stride along N: lane%8 owns 8 consecutive columns, lane/8 strides K
//             by 4; partial sums of the 4 K groups are combined with two shuffles.
// ----------------------------------------------------------------------------
template <typename TA, typename RA, typename TB, typename RB, bool B_KMAJOR, int CW, typename Epi, typename Params>
__device__ __forceinline__ void gemv(Ctx& c, const Params& P, const TA* a, int64_t a_ks, const TB* B, int64_t b_ld,
                                     int N, int K, int64_t item_base) {
    constexpr int kWarps = kThreads / 32;
    if constexpr (B_KMAJOR) {
        const int64_t items = (N + kWarps - 1) / kWarps;
        for (int64_t it = first_item(item_base); it < items; it += gridDim.x) {
            const int n = static_cast<int>(it) * kWarps + c.warp;
            float acc = 0.0f;
            if (n < N) {
                const TB* col = B + static_cast<int64_t>(n) * b_ld;
                for (int k = c.lane * 8; k < K; k += 256) {
                    const int nvalid = min(8, K - k);
                    float av[8], bv[8];
                    ld_row_strided<8>(a + static_cast<int64_t>(k) * a_ks, a_ks, nvalid, av);
                    ld_row<8>(col + k, nvalid, bv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc = fmaf(RA::rnd(av[e]), RB::rnd(bv[e]), acc);
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (n < N && c.lane == 0) Epi::template run<1>(P, 0, n, 1, &acc);
        }
    } else {
        // A warp covers CW columns (64: eight lanes side by side, four K groups; 8: one lane per row
        // piece, 32 K groups -- the latency-friendly shape for a small matrix, which then spreads over
        // eight times as many warps with an eighth of the loads per lane).
        static_assert(CW == 64 || CW == 8, "columns per warp");
        constexpr int kLanesPerRow = CW / 8, kGroups = 32 / kLanesPerRow;
        const int64_t items = (N + CW * kWarps - 1) / (CW * kWarps);
        for (int64_t it = first_item(item_base); it < items; it += gridDim.x) {
            const int n0 = (static_cast<int>(it) * kWarps + c.warp) * CW + (c.lane % kLanesPerRow) * 8;
            float acc[8] = {};
            if (n0 < N) {
                const int nvalid = min(8, N - n0);
#pragma unroll 4
                for (int k = c.lane / kLanesPerRow; k < K; k += kGroups) {
                    float b[8];
                    ld_row<8>(B + static_cast<int64_t>(k) * b_ld + n0, nvalid, b);
                    const float av = RA::rnd(to_f32(a[static_cast<int64_t>(k) * a_ks]));
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(av, RB::rnd(b[e]), acc[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
#pragma unroll
                for (int o = kLanesPerRow; o < 32; o <<= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
            }
            if (n0 < N && c.lane < kLanesPerRow) Epi::template run<8>(P, 0, n0, min(8, N - n0), acc);
        }
    }
}

}  // namespace tk
