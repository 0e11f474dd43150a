/*
 * tm.h - the C ABI of libtmcuda.
 *
 * libtmcuda is a CUDA (sm_100a) implementation of the two hot kernels of
 * triton-metal - the tl.dot matmul and FlashAttention-2 forward/backward -
 * behind that project's handle-based `tm_*` C ABI (plus the five one-dimensional
 * kernels that project's own ABI tests launch: copy_kernel, add_kernel, mul_kernel,
 * scale_bias_kernel, softmax_kernel).  The 23 `tm_*` functions
 * below have the signatures the reference's ctypes shim binds
 * (python/triton_metal/_core.py:70-100); each comment names the reference
 * export it replaces.  Everything prefixed `tmx_` is additive: the reference
 * has no counterpart, and no `tm_*` signature depends on it.
 *
 * Conventions (Sources/TritonMetalCore/Compiler.swift:172-177):
 *   - a returned `char*` is malloc'd; the caller releases it with tm_free;
 *   - handle-returning calls give 0 on failure, status calls give -1;
 *   - the reason for the most recent failure is read (and cleared) by
 *     tm_last_error, which returns "no error" when nothing is stored;
 *   - handles are int64 values from one process-wide table, the first is 1;
 *   - no call throws, aborts or longjmps across the boundary.
 */
#ifndef TM_H
#define TM_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- strings, errors, device ------------------------------------------- */

/* "0.0.1".  Replaces tm_version, Compiler.swift:180-183. */
char *tm_version(void);
/* free() for strings this library returned.  Replaces tm_free, Compiler.swift:185-188. */
void tm_free(void *ptr);
/* Take and clear the last error.  Replaces tm_last_error, Compiler.swift:456-459. */
char *tm_last_error(void);
/* 1 when a CUDA device is present.  Replaces tm_is_active, Runtime.swift:295-298. */
int32_t tm_is_active(void);
/* 1 when the selected device runs sm_100a code (probe kernel launched once and
 * cached).  Replaces tm_is_usable, Runtime.swift:305-308. */
int32_t tm_is_usable(void);
/* Why tm_is_usable is 0, or NULL.  Replaces tm_unusable_reason, Runtime.swift:312-315. */
char *tm_unusable_reason(void);
/* Device name, or NULL without a device.  Replaces tm_device_name, Runtime.swift:318-321. */
char *tm_device_name(void);

/* ---- "compiler": Triton IR text -> kernel descriptor -------------------- */

/* Scan the tt.func signature (and the first tt.dot / rank-2 tensor type) of
 * `ttir` and return a kernel descriptor text - not MSL, and not a compiler:
 * the kernels are precompiled sm_100a functions selected by entry name and
 * element type (for the one-dimensional kernels BLOCK is the extent of the first
 * tt.make_range, and a body that is not the named computation is refused).  `num_simdgroups` is accepted for signature compatibility and
 * only echoed into threads_per_threadgroup.  NULL on failure.
 * Replaces tm_emit_msl, Compiler.swift:192-210. */
char *tm_emit_msl(const char *ttir, int32_t num_simdgroups);
/* Launch metadata as JSON: {"kernels":[{"name","block_size","block_shape",
 * "threads_per_threadgroup","args":[{"index","kind","dtype"}]}]}.
 * Replaces tm_kernel_info, Compiler.swift:214-232 (JSON shape :146-170). */
char *tm_kernel_info(const char *ttir, int32_t num_simdgroups);
/* Turn a descriptor returned by tm_emit_msl into a library handle.
 * Replaces tm_compile_msl, Compiler.swift:235-247. */
int64_t tm_compile_msl(const char *source);
/* The cached-binary path.  The image is either the bytes of a descriptor (the text tm_emit_msl
 * returned) or a binary of this platform - a cubin (ELF) or a fatbin holding sm_100a code.  A
 * binary is loaded as it is: tm_load_kernel looks its entry points up by name (declare them
 * extern "C"), and tm_launch passes argument i to parameter i - a buffer as its device address,
 * i32 / f32 / i64 in their own width - on a grid of (x, y, z) blocks of `threads` threads, after
 * checking count and widths against what the image declares; tm_kernel_max_threads reports the
 * entry point's own limit.  So a caller's own CUDA kernels run behind the same calls as the
 * library's, as arbitrary Metal kernels do behind the reference's.
 * Replaces tm_load_metallib, Compiler.swift:250-263. */
int64_t tm_load_metallib(const void *bytes, int64_t length);
/* Replaces tm_release_library, Compiler.swift:383-386. */
int32_t tm_release_library(int64_t library);

/* ---- runtime ------------------------------------------------------------ */

/* Bind `name` in `library` to its precompiled function.  Unknown names fail with
 * "kernel 'x' not found in library (available: ...)".
 * Replaces tm_load_kernel, Compiler.swift:266-281. */
int64_t tm_load_kernel(int64_t library, const char *name);
/* 1024, or -1.  Replaces tm_kernel_max_threads, Compiler.swift:284-293. */
int64_t tm_kernel_max_threads(int64_t kernel);
/* Replaces tm_release_kernel, Compiler.swift:378-381. */
int32_t tm_release_kernel(int64_t kernel);
/* Allocate `nbytes` of memory that both the host and the GPU address (CUDA
 * managed memory, resident on the device until the host touches it).
 * nbytes <= 0 is an error.  Replaces tm_alloc_buffer, Compiler.swift:296-304. */
int64_t tm_alloc_buffer(int64_t nbytes);
/* Host-addressable pointer to the buffer, valid until tm_free_buffer.
 * Replaces tm_buffer_contents, Compiler.swift:307-315. */
void *tm_buffer_contents(int64_t buffer);
/* Replaces tm_buffer_length, Compiler.swift:317-325. */
int64_t tm_buffer_length(int64_t buffer);
/* Bounds-checked host -> buffer copy.  Replaces tm_buffer_write, Compiler.swift:328-335. */
int32_t tm_buffer_write(int64_t buffer, int64_t offset, const void *source, int64_t length);
/* Bounds-checked buffer -> host copy.  Replaces tm_buffer_read, Compiler.swift:338-348. */
int32_t tm_buffer_read(int64_t buffer, int64_t offset, void *destination, int64_t length);
/* Replaces tm_free_buffer, Compiler.swift:373-376. */
int32_t tm_free_buffer(int64_t buffer);
/* Run `kernel` and wait for it.  Argument i is tt.func argument i; kinds:
 * 0 buffer handle, 1 i32 (low 32 bits), 2 f32 bit pattern (low 32 bits), 3 i64.
 * grid_x/grid_y keep the reference's meaning (one program per block of the
 * descriptor's BLOCK shape; grid_y is batch*heads for the attention kernels):
 * rows or columns beyond grid*BLOCK are not computed, exactly as if those
 * programs had not been dispatched.  The CUDA kernels choose their own CTA
 * shape.  Replaces tm_launch, Compiler.swift:403-448 + Runtime.swift:195-243. */
int32_t tm_launch(int64_t kernel, int64_t grid_x, int64_t grid_y, int64_t grid_z,
                  int64_t threads_per_threadgroup, const int32_t *kinds,
                  const int64_t *values, int32_t arg_count);
/* Replaces tm_live_handle_count, Compiler.swift:451-454. */
int64_t tm_live_handle_count(void);

/* ---- additive entry points (no counterpart in the reference) ------------- */

/* Select the CUDA device for this process (one process per GPU).  Must come
 * before the first allocation or launch; default is $TMCUDA_DEVICE or 0. */
int32_t tmx_set_device(int32_t ordinal);
int32_t tmx_get_device(void);
/* Number of streaming multiprocessors of the selected device, or -1. */
int32_t tmx_sm_count(void);
/* Set an integer option on a loaded kernel.  Known options: "causal" (attention
 * kernels: mask key j > query i), "path" (0 = automatic, 1 = force the generic
 * SIMT kernel, 2 = require a tensor-core kernel - tcgen05 for 16-bit elements,
 * 3xTF32 for fp32 - and fail if the shape is not eligible).  0 / -1. */
int32_t tmx_kernel_set_option(int64_t kernel, const char *name, int64_t value);
/* Which implementation the most recent launch of `kernel` used:
 * 0 none yet, 1 generic SIMT, 2 tcgen05.  -1 on a bad handle. */
int32_t tmx_kernel_last_path(int64_t kernel);
/* tm_launch without the wait: enqueue on the library's stream and return. */
int32_t tmx_launch_async(int64_t kernel, int64_t grid_x, int64_t grid_y, int64_t grid_z,
                         int64_t threads_per_threadgroup, const int32_t *kinds,
                         const int64_t *values, int32_t arg_count);
/* Enqueue `repeats` back-to-back launches between two CUDA events on the
 * library's stream, wait, and store the elapsed milliseconds for all of them in
 * *elapsed_ms (the reference packs `repeats` dispatches into one command buffer
 * the same way: Sources/TritonMetalBench/GEMMBenchmark.swift:256-277). */
int32_t tmx_launch_timed(int64_t kernel, int64_t grid_x, int64_t grid_y, int64_t grid_z,
                         int64_t threads_per_threadgroup, const int32_t *kinds,
                         const int64_t *values, int32_t arg_count, int32_t repeats,
                         float *elapsed_ms);
/* Wait for everything enqueued on the library's stream; surfaces device-side
 * status words (bounded waits that gave up) as -1. */
int32_t tmx_synchronize(void);
/* Asynchronous copies (host memory should be pinned).  A write runs on an upload stream of the
 * library's own: it starts as soon as the last launch that took the buffer as an argument (and
 * any read-back of the buffer still in flight) has finished - not behind every kernel enqueued
 * before it - and everything enqueued after it sees the new contents, so the upload of the next
 * piece of input overlaps the kernels working on the current one while each buffer still sees
 * the order of the calls.  A read starts after everything enqueued before it but runs on a side
 * stream, so it overlaps the writes and launches enqueued after it; a later launch or write that
 * takes the same buffer waits for the read-back.  tmx_synchronize, tmx_timer_end and every
 * blocking tm_* call wait for the uploads and read-backs too.  tmx_matmul_gathered and
 * tmx_matmul_f32_static do not look for read-backs in flight: synchronise before handing them a
 * buffer that tmx_buffer_read_async is still reading. */
int32_t tmx_buffer_write_async(int64_t buffer, int64_t offset, const void *source, int64_t length);
int32_t tmx_buffer_read_async(int64_t buffer, int64_t offset, void *destination, int64_t length);
/* Fill `length` bytes of the buffer with `byte` (asynchronous). */
int32_t tmx_buffer_fill(int64_t buffer, int64_t offset, int32_t byte, int64_t length);
/* Event pair on the library's stream: begin/end bracket a timed region. */
int32_t tmx_timer_begin(void);
int32_t tmx_timer_end(float *elapsed_ms);
/* Count of kernels this library has launched since load (for launch accounting). */
int64_t tmx_launch_count(void);

/* A buffer of plain device memory (no host pointer: tm_buffer_contents fails on it), for
 * buffers handed to other device-side libraries such as NCCL.  0 on failure. */
int64_t tmx_alloc_device_buffer(int64_t nbytes);
/* The library's stream as a cudaStream_t, for enqueuing other stream-ordered work (an NCCL
 * collective, a torch op through an external-stream wrapper) in order with the launches.
 * NULL on failure. */
void *tmx_stream_handle(void);
/* The device address of any buffer, for interop with libraries that take raw pointers. */
void *tmx_buffer_device_pointer(int64_t buffer);

/* fp32 C[M,N] = A[M,K] @ B[K,N] for callers that must not allocate device memory.
 * No counterpart in the reference.
 *
 * The fp32 matmul runs on the tensor cores as 3xTF32, which needs scratch for the split
 * operands: 8*(M+N)*roundup(K,4) bytes.  tm_launch takes that from a workspace it grows with
 * cudaMalloc when a larger problem arrives.  That is unusable for a host that has already
 * given all device memory to its own pool, for a service that may not allocate once it has
 * started serving, and for any code running where the CUDA runtime refuses allocation.  This
 * entry point is the same kernel pair with the scratch in a fixed array that is part of the
 * library image: it calls no cudaMalloc, cudaFree or other allocating routine.
 *
 *  - a, b, c are fp32 buffer handles (the caller still owns inputs and outputs); strides are
 *    in elements, any non-negative value; the call waits for the result like tm_launch.
 *  - Limit: 8*(M+N)*roundup(K,4) must not exceed tmx_matmul_f32_static_capacity() (8 MiB;
 *    e.g. 512 x 512 x 1024).  Larger problems, and problems below 128 x 64 x 32, are refused
 *    with -1 and a message; use tm_launch for those.
 *  - Every GPU that loads the library holds the 8 MiB array until the process exits.
 *  - The first call on a device looks up the array's device address (one
 *    cudaGetSymbolAddress with that device current).  Make that first call during start-up,
 *    before any stream capture is begun.
 *  - "Allocates nothing" is a statement about calls, not about loading: the CUDA runtime loads
 *    a module lazily, and the module that holds the array and these kernels is loaded by that
 *    first address lookup (or first launch) - that is when the driver sets aside the 8 MiB and
 *    the kernel images on the GPU.  A host that is about to hand all remaining device memory to
 *    its own pool must therefore make the first call, or tmx_matmul_f32_static_prepare, before
 *    it does so; a first call made afterwards can fail for lack of memory.  From the second
 *    call on, free device memory is the same before and after a call.
 *  - All calls share the one array and it keeps whatever the last call left in it.  Nothing
 *    needs clearing: each call first rewrites every word its GEMM reads.  Calls are ordered on
 *    the library's single stream; work that overlaps on the GPU with one of these calls and
 *    also uses the array (there is none inside this library) would race. */
int32_t tmx_matmul_f32_static(int64_t a, int64_t b, int64_t c, int64_t M, int64_t N, int64_t K,
                              int64_t stride_am, int64_t stride_ak, int64_t stride_bk,
                              int64_t stride_bn, int64_t stride_cm, int64_t stride_cn);
/* Size in bytes of the fixed scratch array behind tmx_matmul_f32_static. */
int64_t tmx_matmul_f32_static_capacity(void);
/* The once-per-device set-up of tmx_matmul_f32_static without a matmul: resolves the array's
 * address and thereby loads the module that holds it.  0 / -1.  No counterpart in the reference. */
int32_t tmx_matmul_f32_static_prepare(void);
/* Free and total device memory in bytes, as the driver reports them.  0 / -1. */
int32_t tmx_device_memory(int64_t *free_bytes, int64_t *total_bytes);

/* ---- row-sharded matmul over several GPUs (no counterpart in the reference: it drives one
 * device, Sources/TritonMetalCore/Runtime.swift:10-11) -------------------------------------
 *
 * One process per GPU.  Each rank computes a block of rows of C = A @ B (B replicated) and
 * every rank ends up with the whole C.  Instead of a collective behind the kernel, the
 * kernel's epilogue stores each finished tile into every rank's copy of C - its own and,
 * through memory mapped from the other processes, the peers' - so the exchange overlaps the
 * main loop.  Set-up, once: every rank allocates its copy of C and a flag array
 * (tmx_alloc_device_buffer; tmx_gather_flag_bytes() bytes, zero-filled), exports both
 * (tmx_ipc_export), passes the 64-byte tokens to the other ranks by any means, and imports
 * theirs (tmx_ipc_import). */

/* The token for another process to map `buffer` (plain device memory only).  0 / -1. */
int32_t tmx_ipc_export(int64_t buffer, void *handle64);
/* Map another process's buffer of `nbytes` bytes; enables peer access to its GPU.  A buffer
 * handle (device-only; tm_free_buffer unmaps it), 0 on failure. */
int64_t tmx_ipc_import(const void *handle64, int64_t nbytes);
/* Size of a flag array in bytes (64 slots x 8 ranks x 4). */
int64_t tmx_gather_flag_bytes(void);
/* Enqueue C[row0 : row0+rows, :] = A[rows, K] @ B[K, N] (16-bit, row-major, dense) on the
 * tensor cores and store the result rows into every copy c_replicas[0..world-1] of the whole
 * C (c_replicas[rank] is this rank's own buffer, the others are imported).  When this rank's
 * last tile is out it writes `epoch` into word slot*8 + rank of every peer's flag array; with
 * wait_for_peers != 0 the kernel then waits (bounded; on expiry the launch fails like any
 * other bounded wait) until words slot*8 + r of its own flag array have reached `epoch` for all
 * r, so that on completion this rank's copy of C holds every rank's rows.
 *  - `epoch` must be positive and grow from launch to launch on the same slot, on all ranks
 *    alike; slots 0...63 let independent row blocks be in flight at once.
 *  - All ranks must make the matching call; a rank that does not lets the others' waits run out.
 *  - A later launch overwrites the peers' copies: the caller makes sure (a barrier, or a second
 *    set of copies) that every rank is done reading C before any rank computes into it again.
 * Returns 0 / -1 at once; tmx_synchronize or any blocking call waits for the kernel. */
int32_t tmx_matmul_gathered(int64_t kernel, int64_t a, int64_t b, const int64_t *c_replicas,
                            const int64_t *flag_buffers, int32_t world, int32_t rank, int64_t row0,
                            int64_t rows, int64_t N, int64_t K, int32_t slot, uint32_t epoch,
                            int32_t wait_for_peers);

/* ---- failure-path aids (no counterpart in the reference) -------------------
 *
 * Every wait inside the tensor-core kernels is bounded: when its cycle budget runs out the
 * kernel records where in a host-visible status word and returns, and the next call that
 * synchronises (tm_launch, tm_buffer_read/write, tmx_synchronize, tmx_timer_end) returns -1
 * with "a bounded wait gave up inside the kernel ..." and clears the word.  These two entry
 * points let a test suite walk that path without breaking a kernel. */

/* Launch a small kernel that waits - with the same bounded waits and `budget_cycles` (1...2e9)
 * - on a barrier nothing arrives on, and wait for it.  The waits run out, the kernel records
 * that and returns normally (no trap, the context stays usable).  results[0] (a wait by one
 * thread) and results[1] (a wait by a whole warp) are 1 when the wait reported "gave up".
 * The status word is left set: the next synchronising call returns -1. */
int32_t tmx_selftest_bounded_wait(int64_t budget_cycles, int32_t *results);
/* The per-CTA work lists the persistent attention kernels walk for a problem shape (kind 0
 * forward: 256-row query blocks; 1 dq, 2 dkdv: 128-row tiles), for inspection and tests.  Up to
 * `capacity` (batch-head, block) pairs go to items_out, ctas + 1 list offsets to begin_out, the
 * modelled cost of every CTA to load_out (each may be NULL; a list never has more CTAs than
 * items, so fewer than `ctas` + 1 offsets may be written).  Returns the item count or -1. */
int64_t tmx_debug_attention_schedule(int32_t kind, int32_t bh, int32_t rows, int32_t n_ctx, int32_t causal,
                                     int32_t ctas, int32_t *items_out, int64_t capacity, int32_t *begin_out,
                                     int64_t *load_out);
/* Set the device status word from the host, as a kernel whose wait gave up would. */
int32_t tmx_debug_inject_status(int32_t code, int32_t where, int32_t block, int32_t extra);

#ifdef __cplusplus
}
#endif
#endif /* TM_H */
