/* mlcb -- C ABI of the B200 kernel backend for the mlc inference compiler.
 *
 * This is the boundary the executor launches generated kernels through.  It
 * takes the place of the reference's Triton runtime: where
 * mlc/runtime/triton_runtime.py writes a Python module, imports it and calls
 * `fn[grid](*tensors, **constants)`, a host binds these entry points instead:
 * compile one CUDA translation unit for sm_100a, load the image, look kernels up
 * by name, and enqueue them on a caller-supplied stream.
 *
 * Conventions
 *   - every function returns 0 on success, or a non-zero CUresult / nvrtcResult
 *     (NVRTC codes are offset by MLCB_NVRTC_BASE); nothing throws, nothing exits;
 *     mlcb_last_error() gives a human-readable message for the calling thread;
 *   - the library owns CUmodule / CUfunction handles only.  It never allocates,
 *     frees or retains device memory: pointers are whatever the host's tensors
 *     hold, captured once when a launch is bound;
 *   - mlcb_launch / mlcb_launch_many do not synchronise, allocate or load
 *     anything, so they are legal inside CUDA stream capture;
 *   - shapes, strides and vector widths are literals in the generated source, so
 *     a launch carries only buffer base pointers (inputs first, then outputs),
 *     the same contract as the reference's generated Triton
 *     (mlc/codegen/triton_backend.py:9-13);
 *   - distinct modules may be used from distinct threads; one module is used from
 *     one thread at a time.
 */
#ifndef MLCB_H
#define MLCB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLCB_ABI_VERSION 1
#define MLCB_NVRTC_BASE 100000
#define MLCB_ERR_LIBRARY 200001 /* libcuda / libnvrtc could not be loaded */
#define MLCB_ERR_ARGUMENT 200002

/* launch flags */
#define MLCB_LAUNCH_DEPENDENT 1u /* programmatic stream serialisation (PDL) */

typedef struct mlcb_module mlcb_module;
typedef struct mlcb_kernel mlcb_kernel;

/* One entry of a batched enqueue (mlcb_launch_many). */
typedef struct mlcb_launch_desc {
    mlcb_kernel* kernel;
    uint32_t grid_x;
    uint32_t block_x;
    uint32_t smem_bytes;
    uint32_t flags;
    const uint64_t* device_ptrs;
    int32_t nptrs;
    int32_t reserved;
} mlcb_launch_desc;

/* ABI version of the loaded library (MLCB_ABI_VERSION at build time). */
int mlcb_version(void);

/* Message for the most recent failure on the calling thread ("" if none). */
const char* mlcb_last_error(void);

/* Source -> device image.  Replaces write_module + the Triton JIT
 * (mlc/runtime/triton_runtime.py:36-44 and the lazy compile at first launch).
 * `arch` is e.g. "sm_100a"; `opts` are extra NVRTC options.  On success *image
 * is a malloc'd cubin of *size bytes, released with mlcb_free_image.  The
 * compiler log (warnings or errors) is copied into `log`, NUL-terminated and
 * truncated to logcap. */
int mlcb_compile(const char* src, const char* arch, const char* const* opts, int nopts,
                 void** image, size_t* size, char* log, size_t logcap);
void mlcb_free_image(void* image);

/* Image -> loaded module in the primary context of `device`.  Replaces
 * load_module (mlc/runtime/triton_runtime.py:47-57). */
int mlcb_module_load(const void* image, size_t size, int device, mlcb_module** out);
int mlcb_module_unload(mlcb_module* m);

/* Kernel lookup by symbol.  Replaces `getattr(self.module, k.name)`
 * (mlc/runtime/triton_runtime.py:76). The handle lives as long as its module. */
int mlcb_get_kernel(mlcb_module* m, const char* name, mlcb_kernel** out);

/* Registers per thread, static shared memory and the largest legal block of a
 * loaded kernel (for reports; no reference counterpart). */
int mlcb_kernel_info(mlcb_kernel* k, int* regs, int* static_smem, int* max_threads);

/* Enqueue one kernel: `fn[grid](*args, **consts)` at
 * mlc/runtime/executor.py:194-196 and mlc/runtime/triton_runtime.py:92-97.
 * `stream` is a cudaStream_t / CUstream value (0 = legacy default stream). */
int mlcb_launch(mlcb_kernel* k, uint32_t grid_x, uint32_t block_x, uint32_t smem_bytes,
                const uint64_t* device_ptrs, int nptrs, uint64_t stream, uint32_t flags);

/* Enqueue a run of kernels in order with one call across the boundary; stops at
 * the first failure and returns its code (*failed_at = its index, if given).
 * Replaces the interpreter loop over consecutive generated kernels in
 * run_kernels (mlc/runtime/executor.py:186-202). */
int mlcb_launch_many(const mlcb_launch_desc* descs, int n, uint64_t stream, int* failed_at);

#ifdef __cplusplus
}
#endif
#endif /* MLCB_H */
