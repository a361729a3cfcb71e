/* C ABI of libtrainkernel_rt.so: load and launch one generated training-step kernel.
 *
 * This is the native boundary of the compiled-step path.  In the reference the
 * same boundary is a pybind11 module that is generated and compiled together
 * with every kernel and exposes `launch(inputs, outputs, workspace)` and
 * `resource_usage()` (reference: trainkernel/codegen.py:862-896, called from
 * trainkernel/runtime.py:39-43 and :96).  Here it is one prebuilt shared library
 * over the CUDA driver API with plain pointers and sizes in every signature; it
 * has no PyTorch, pybind11 or CUDA-runtime dependency and resolves libcuda.so.1
 * lazily, so it can be loaded (not launched) on a machine without a driver.
 *
 * Conventions: every function returns 0 on success, otherwise a CUresult value
 * or one of the TK_E_* codes below; nothing throws; tk_last_error() returns a
 * thread-local description of the most recent failure on the calling thread.
 * tk_module_launch never synchronises and never allocates, so it may be called
 * while the stream is being captured into a CUDA graph.
 */
#ifndef TRAINKERNEL_RT_H
#define TRAINKERNEL_RT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TK_E_ARGUMENT 100001   /* null pointer, bad count, bad size */
#define TK_E_DRIVER   100002   /* libcuda.so.1 or one of its entry points is missing */
#define TK_E_CAPACITY 100003   /* grid larger than what can be co-resident */
#define TK_E_KERNEL   100004   /* the kernel reported a timed-out wait; see tk_module_status */

typedef struct tk_module tk_module;   /* owns CUmodule/CUfunction, barrier words, status words */

/* Where a tensor map's base pointer comes from at launch time. */
enum { TK_BASE_INPUT = 0, TK_BASE_OUTPUT = 1, TK_BASE_WORKSPACE = 2 };

/* Recipe for one 2-D, 128-byte-swizzled tiled tensor map over 16-bit elements. */
typedef struct {
    int32_t base_kind;            /* TK_BASE_* */
    int32_t base_index;           /* input / output index; ignored for the workspace */
    uint64_t byte_offset;         /* added to the base pointer */
    uint64_t inner;               /* extent of the unit-stride dimension, in elements */
    uint64_t outer;               /* extent of the other dimension */
    uint64_t outer_stride_bytes;  /* multiple of 16 */
    uint32_t box_inner;           /* 64 */
    uint32_t box_outer;           /* <= 256 */
    uint32_t element_bytes;       /* 2 */
    uint32_t reserved;
} tk_tensor_map_desc;

/* Load a cubin and look up `entry`.  Replaces the per-kernel pybind module build
 * (reference: trainkernel/runtime.py:143-152).  `threads` and `dynamic_smem` are the launch
 * geometry the kernel was generated for; `n_inputs`/`n_outputs` size the pointer tables in the
 * kernel parameter block (at least one slot each is always laid out). */
int tk_module_load(const void* cubin, size_t cubin_bytes, const char* entry, int device,
                   int threads, size_t dynamic_smem, int n_inputs, int n_outputs,
                   const tk_tensor_map_desc* maps, int n_maps, tk_module** out);

/* Cooperative launch on `stream` (a CUstream / cudaStream_t).  Replaces `launch()`
 * (reference: trainkernel/codegen.py:863-888).  Pointers are borrowed for the call only. */
int tk_module_launch(tk_module* module, const void* const* inputs, void* const* outputs,
                     void* workspace, int grid, void* stream);

/* tk_module_launch with launch flags.  TK_LAUNCH_TRUST_CARRIED tells a kernel that keeps derived values
 * from one launch to the next (the BF16 copies of FP32 master weights, written by the step that updated the
 * masters) that the caller has not modified the in-place state since this module's previous launch, so the
 * kernel may skip recomputing them.  The flag is ignored (the values are recomputed) by the first launch ever,
 * after tk_module_reset / tk_module_invalidate_carried, and by the first launch recorded into each stream
 * capture, so a replayed CUDA graph always starts from the caller's state.  tk_module_launch passes no flags.
 * No counterpart in the reference, which recasts every weight in every step (trainkernel/codegen.py:419-423). */
#define TK_LAUNCH_TRUST_CARRIED 1u
int tk_module_launch_flags(tk_module* module, const void* const* inputs, void* const* outputs,
                           void* workspace, int grid, void* stream, uint32_t flags);

/* Enqueue on `stream` the invalidation of the values carried over between launches (see above): for a
 * caller that rewrites the state by means the host cannot see.  No counterpart in the reference. */
int tk_module_invalidate_carried(tk_module* module, void* stream);

/* Device ordinal the module was loaded on; the workspace size its kernel's plan needs, as recorded by
 * whoever loaded it (0 when never recorded).  Used by launch paths that must check what they are handed.
 * No counterpart in the reference (its launch derives both from the workspace tensor, trainkernel/codegen.py:866). */
int tk_module_device(tk_module* module, int* out);
/* Launches issued through this module so far, by any caller in the process: lets a caller that tracks
 * carried values notice that somebody else launched the kernel in between.  No counterpart in the reference. */
int tk_module_launches(tk_module* module, uint64_t* out);
int tk_module_set_workspace_bytes(tk_module* module, size_t bytes);
/* Declares which base pointers the module's kernel accesses with 16-byte vector loads and stores:
 * `inputs[i]` / `outputs[i]` non-zero for kernel input / output i (arrays may be shorter than the kernel's
 * lists), `workspace` non-zero for the workspace.  Every later launch returns TK_E_ARGUMENT instead of
 * launching when one of them is not 16-byte aligned.  Call it once, before the first launch.  No counterpart
 * in the reference, whose generated kernels use scalar accesses throughout (trainkernel/codegen.py:419-423). */
int tk_module_require_alignment(tk_module* module, const uint8_t* inputs, int n_inputs, const uint8_t* outputs, int n_outputs, int workspace);
int tk_module_workspace_bytes(tk_module* module, size_t* out);

/* {registers per thread, local bytes per thread, static + dynamic shared bytes per block,
 * resident blocks per SM}.  Replaces `resource_usage()` (reference: trainkernel/codegen.py:889-895). */
int tk_module_resource_usage(tk_module* module, int64_t out[4]);

/* Launch the kernel with thread-block clusters of `size` CTAs (1, 2, 4 or 8).  Kernels generated with
 * the two-CTA tcgen05 GEMM need 2; kernels whose stages end in the hardware cluster barrier are
 * launched as ONE cluster (grid == size).  Recomputes the co-resident capacity for clustered launches.
 * New on this back end: the reference's kernels have no cluster dimension (trainkernel/codegen.py:886). */
int tk_module_set_cluster(tk_module* module, int size);

/* Launch with (1, the default) or without (0) the cooperative-launch attribute.  A kernel that runs as
 * ONE cluster is co-scheduled by the cluster itself and does not need it.  A grid-barrier kernel
 * launched without it relies on the grid fitting the idle device (the capacity check of
 * tk_module_launch still applies, and every wait in the kernel is bounded): meant for hardware
 * profilers that cannot replay cooperative launches.  No counterpart in the reference, whose launches
 * are always cooperative (trainkernel/codegen.py:886). */
int tk_module_set_cooperative(tk_module* module, int enabled);

/* Launch with (1) or without (0, the default) programmatic stream serialisation: the kernel may then START
 * while its predecessor on the stream is still finishing, and sets up what needs no memory (barriers in
 * shared memory, tensor memory, tensor-map prefetch) before it waits, inside the kernel
 * (`griddepcontrol.wait`), for the predecessor to complete and its writes to be visible.  The generated
 * kernels always contain that wait, which does nothing in an ordinary launch.  It takes the launch latency
 * and the prologue of a step off the critical path of back-to-back steps (a CUDA graph of steps, an eager
 * loop).  No counterpart in the reference (trainkernel/codegen.py:886). */
int tk_module_set_early_launch(tk_module* module, int enabled);

/* Largest grid a cooperative launch of this kernel accepts on its device. */
int tk_module_max_coresident_blocks(tk_module* module, int* out);

/* Synchronise `stream`, then copy the kernel's status words {code, stage, block, detail}.
 * Returns TK_E_KERNEL when code != 0; from then on every launch of this module is refused with TK_E_KERNEL
 * until tk_module_reset, because a kernel that gave up on a wait leaves partial outputs behind and later
 * launches would give up early too.  The status words are sticky on the device, so callers of a long loop
 * should poll this every few steps.  (The reference cannot report a stuck barrier:
 * cooperative_groups grid.sync() has no timeout, reference: trainkernel/codegen.py:833-836.) */
int tk_module_status(tk_module* module, void* stream, uint32_t out[4]);

/* Clear status and barrier words after an error (synchronises the device context). */
int tk_module_reset(tk_module* module);

/* Upper bound, in nanoseconds, for any single wait inside the kernel (default 2e9). */
int tk_module_set_timeout(tk_module* module, uint64_t nanoseconds);

/* Override the arrival count the grid barrier waits for; 0 restores gridDim.x.  Only used by
 * tests that make a barrier time out on purpose without hanging the device. */
int tk_module_set_expected_arrivals(tk_module* module, uint32_t arrivals);

/* Synchronise `stream`, then copy up to `count` (at most 256) 64-bit stamps written by a kernel generated
 * with stage stamps (the built-in form of the reference's source-patching stage profiler, reference:
 * scripts/profile_stages.py:36-54).  Layout, all %globaltimer nanoseconds unless noted: [0, 64) block 0
 * leaves stage boundary s (entry 0: kernel start, entry `stages`: kernel end); [64, 128) block 0 arrives at
 * grid barrier k; [128, 192) the last block arrives at grid barrier k; [192, 248) nanoseconds block 0 waited
 * for its peers' flags before stage s (multi-GPU kernels); [248, 254) role-level trace of one tile. */
int tk_module_stage_stamps(tk_module* module, void* stream, uint64_t* out, int count);

void tk_module_unload(tk_module* module);

const char* tk_last_error(void);

/* Size of the device-resident workspace that tk_module_launch_static_workspace lends to a kernel. */
#define TK_STATIC_WORKSPACE_BYTES (4u << 20)

/* Like tk_module_launch, but the workspace is a fixed TK_STATIC_WORKSPACE_BYTES array that lives in
 * libtrainkernel_noalloc.so's device image, so neither the caller nor the library allocates.  It has
 * no counterpart in the reference, whose callers always allocate a workspace tensor
 * (trainkernel/runtime.py:58-64).  For callers that must not allocate when they launch a step:
 * `workspace_bytes` is what the kernel's plan needs and is rejected with TK_E_CAPACITY when it exceeds
 * the array; `device` is the ordinal the module was loaded on.  All calls on a device share the one
 * array (overlapping launches race; nothing needs clearing between calls).  The first call on a device
 * looks the array's address up through the CUDA runtime and should happen before any stream capture.
 * On failure a message is written to `error` (may be NULL).  Exported by libtrainkernel_noalloc.so. */
int tk_module_launch_static_workspace(tk_module* module, int device, const void* const* inputs,
                                      void* const* outputs, size_t workspace_bytes, int grid,
                                      void* stream, char* error, size_t error_capacity);

/* Number of kernel launches issued through this library by the calling process. */
uint64_t tk_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
