/*
 * C ABI of the B200 execution backend ("torq_b200"): the surface a HAL driver
 * placed beside the reference's runtime/driver binds to, and the one the tests
 * call. Plain pointers and sizes only; no exceptions cross it; every function
 * returns a status whose numbering equals iree_status_code_t, the convention
 * of the reference driver (runtime/driver/torq_device.c, TorqExecutable.cc).
 *
 * Each entry point names the reference interface it stands in for.
 */
#ifndef TORQ_B200_H_
#define TORQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum tb200_status {
  TB200_OK = 0,
  TB200_CANCELLED = 1,
  TB200_UNKNOWN = 2,
  TB200_INVALID_ARGUMENT = 3,
  TB200_DEADLINE_EXCEEDED = 4,
  TB200_NOT_FOUND = 5,
  TB200_ALREADY_EXISTS = 6,
  TB200_PERMISSION_DENIED = 7,
  TB200_RESOURCE_EXHAUSTED = 8,
  TB200_FAILED_PRECONDITION = 9,
  TB200_ABORTED = 10,
  TB200_OUT_OF_RANGE = 11,
  TB200_UNIMPLEMENTED = 12,
  TB200_INTERNAL = 13,
  TB200_UNAVAILABLE = 14,
  TB200_DATA_LOSS = 15,
};

enum tb200_memory_type {
  TB200_MEMORY_DEVICE_LOCAL = 0, /* HBM, not host visible */
  TB200_MEMORY_HOST_PINNED = 1,  /* HOST_VISIBLE | HOST_COHERENT staging */
};

typedef struct tb200_device tb200_device_t;
typedef struct tb200_executable tb200_executable_t;
typedef struct tb200_buffer tb200_buffer_t;

/* (buffer, offset, length) exactly as iree_hal_buffer_ref_t is consumed at
 * runtime/driver/torq_command_buffer.c:467-499. length 0 = "to end of buffer". */
typedef struct tb200_binding {
  tb200_buffer_t* buffer;
  uint64_t offset;
  uint64_t length;
} tb200_binding_t;

typedef struct tb200_io_info {
  uint32_t dtype; /* enum tb200_dtype */
  uint32_t rank;
  int32_t shape[4];
  uint64_t bytes;
} tb200_io_info_t;

/* Device = iree_hal_torq_device_create (runtime/driver/torq_device.c:80-132);
 * owns one CUDA context binding and one stream. */
int tb200_device_create(int cuda_ordinal, tb200_device_t** out_device);
int tb200_device_destroy(tb200_device_t* device);
/* iree_hal_torq_device_query_i64 (runtime/driver/torq_device.c:194-233):
 * ("hal.executable.format","torq-b200-ops") -> 1, ("hal.device","concurrency") -> 1,
 * ("hal.dispatch","concurrency") -> 1; anything else NOT_FOUND. */
int tb200_device_query_i64(tb200_device_t* device, const char* category, const char* key,
                           int64_t* out_value);
/* The cudaStream_t every transfer and dispatch of this device is queued on, so a
 * caller can record its own events on it or order other work after it (role of the
 * HAL semaphore a queue_execute signals, runtime/driver/torq_device.c:487-526). */
void* tb200_device_stream(tb200_device_t* device);
/* Text of the most recent failure on this device (thread-unsafe convenience). */
const char* tb200_last_error(tb200_device_t* device);
const char* tb200_status_string(int status);

/* Host event log, schema of runtime/torq_hw/src/TorqEventLog.cpp:23-115
 * (dispatch_name,invocation_id,action_id,timestamp_us,event); NULL path stops it.
 * While enabled every op of a dispatch is bracketed by CUDA events. */
int tb200_device_set_profile_csv(tb200_device_t* device, const char* path);

/* Buffers = iree_hal_allocator_allocate_buffer (runtime/driver/torq_allocator.c:182-236). */
int tb200_buffer_alloc(tb200_device_t* device, uint64_t bytes, int memory_type,
                       tb200_buffer_t** out_buffer);
/* Wrap device memory owned by the caller (iree_hal_allocator_import_buffer role). */
int tb200_buffer_import(tb200_device_t* device, void* device_pointer, uint64_t bytes,
                        tb200_buffer_t** out_buffer);
int tb200_buffer_free(tb200_buffer_t* buffer);
/* Stream-ordered transfers (command buffer update/copy, torq_command_buffer.c:332-373).
 * `host` should be pinned for the copy to overlap; pageable memory also works. */
int tb200_buffer_upload(tb200_buffer_t* buffer, uint64_t offset, const void* host, uint64_t bytes);
int tb200_buffer_download(tb200_buffer_t* buffer, uint64_t offset, void* host, uint64_t bytes);
void* tb200_buffer_pointer(tb200_buffer_t* buffer); /* device or pinned-host address */
uint64_t tb200_buffer_size(tb200_buffer_t* buffer);

/* Executable = nop_executable_cache prepare + native_executable create
 * (runtime/driver/nop_executable_cache.cc:93-110, native_executable.cc:41-108,
 * TorqExecutable.cc:655-752): validates the blob (magic/version mismatch ->
 * UNAVAILABLE like the runtime_version check at TorqExecutable.cc:663-667),
 * COPIES what it needs from `bytes`, uploads constants once, plans launches. */
int tb200_executable_create(tb200_device_t* device, const void* bytes, size_t n_bytes,
                            tb200_executable_t** out_executable);
int tb200_executable_destroy(tb200_executable_t* executable);
int tb200_executable_io_count(tb200_executable_t* executable, uint32_t* n_inputs, uint32_t* n_outputs);
int tb200_executable_io_info(tb200_executable_t* executable, int is_output, uint32_t index,
                             tb200_io_info_t* out_info);
uint32_t tb200_executable_op_count(tb200_executable_t* executable);
/* Number of CUDA kernels one dispatch launches. */
uint32_t tb200_executable_launch_count(tb200_executable_t* executable);

/* Dispatch = iree_hal_torq_command_buffer_dispatch
 * (runtime/driver/torq_command_buffer.c:390-508): bindings are inputs first, then
 * outputs; every binding non-NULL (:488-495) and large enough (OUT_OF_RANGE,
 * TorqExecutable.cc:512-531). Asynchronous: work is queued on the device stream. */
int tb200_dispatch(tb200_executable_t* executable, const tb200_binding_t* bindings, size_t n_bindings);
/* Host wait with a deadline (TorqHw::wait, runtime/torq_hw/src/TorqHw.cpp:155-213):
 * DEADLINE_EXCEEDED when the stream has not drained in time. ABORTED when a kernel gave up one of
 * its bounded internal waits (the message names which): the device stays usable, the results of
 * the dispatches since the last successful wait are undefined, and an executable that runs as one
 * persistent kernel (a decode step) must be destroyed and created again, since its barrier
 * counters no longer match. */
int tb200_wait(tb200_device_t* device, uint64_t timeout_ns);

/* The reference's synchronous host-pointer dispatch (the command buffer maps every
 * binding to a host pointer, torq_command_buffer.c:467-499, then
 * TorqExecutable::executeDispatch copies in, runs, copies out,
 * TorqExecutable.cc:1025-1125): H2D of every input, dispatch, D2H of every
 * output, wait. Host pointers may be pageable or pinned. */
int tb200_invoke_host(tb200_executable_t* executable, const void* const* host_inputs,
                      void* const* host_outputs);
/* The same call without the final wait (the deferred command buffer + queue_execute form of
 * the reference, runtime/driver/torq_device.c:393-442,487-526): uploads go to a second
 * stream into one of two staging sets, so the upload of call k+1 overlaps the kernels of
 * call k. Host input memory must stay valid, and host output memory is defined, only after
 * tb200_wait() returns; pinned host memory is needed for the overlap. */
int tb200_invoke_host_async(tb200_executable_t* executable, const void* const* host_inputs,
                            void* const* host_outputs);

/* Per-op device time of one dispatch (CUDA events around each op, averaged over
 * `iters` runs after `warmup`); ms[op_count]. Profiling aid; role of the per-action
 * event log at TorqExecutable.cc:1030-1099. */
int tb200_executable_profile_ops(tb200_executable_t* executable, const tb200_binding_t* bindings,
                                 size_t n_bindings, int warmup, int iters, float* ms,
                                 uint32_t ms_capacity);
/* Name of the kernel the plan picked for op `index` (static string). */
const char* tb200_executable_op_kernel(tb200_executable_t* executable, uint32_t index);

/* ---- tensor-parallel groups (LLM decode split over the GPUs of one node) ----
 * The reference's device offers no collectives (create_channel and the collective commands are
 * UNIMPLEMENTED, runtime/driver/torq_device.c:235-240): these three calls are what a HAL channel
 * for this backend would be built on. An executable whose op list holds TB200_OP_ALLREDUCE ops is
 * one shard of a group (rank and size are read from the ops). One process per GPU: each member
 * asks for its handle, the handles travel out of band (any host transport), and every member
 * connects with the full, rank-ordered list before its first dispatch. From then on a dispatch
 * must be made by every member: the decode-step kernels of the members exchange their partial
 * results through each other's memory (peer stores) and wait for one another (bounded: a member
 * that never shows up ends the others' dispatch with TB200_ABORTED from tb200_wait). */
typedef struct tb200_comm_handle_t { unsigned char bytes[96]; } tb200_comm_handle_t;
int tb200_executable_comm_info(tb200_executable_t* executable, int32_t* rank, int32_t* group_size);
int tb200_executable_comm_handle(tb200_executable_t* executable, tb200_comm_handle_t* out);
int tb200_executable_connect_peers(tb200_executable_t* executable, const tb200_comm_handle_t* handles, size_t n);

/* No counterpart in the reference. The split-K int8-weight GEMV (y[b,n] = scale[n] * sum_k
 * x[b,k] * W[n,k]; x bf16 [B,K], W int8 [N,K], scale bf16 [N], y bf16 or fp32 [B,N]) for
 * callers that cannot allocate: a host whose own allocator already holds all device memory,
 * or a latency-critical loop that cannot afford the device-wide synchronisation an
 * allocation may bring. Its partial sums live in a fixed 4 MiB array inside the library
 * (held by every GPU that loads the library until the process exits), so
 * slices * B * N must be <= 1,048,576 or the call returns TB200_OUT_OF_RANGE (and says so on
 * stderr); so does a slice count that leaves K slices longer than 2048 values at B >= 3. x and W
 * must be 16-byte aligned, y and scale aligned to their element (else TB200_INVALID_ARGUMENT).
 * The calling thread's current device is left as it was. All pointers are device pointers on GPU `cuda_ordinal`; `stream` is a
 * cudaStream_t or NULL; splits <= 0 picks the slice count. The first call on a device
 * resolves the array's device address and should be made before any stream capture. Calls
 * share the array: calls that may overlap on the GPU race with each other and must be ordered
 * by the caller. Nothing is allocated or freed by this call. */
int tb200_gemv_w8_noalloc(int cuda_ordinal, void* stream, const void* x_bf16, const void* w_i8,
                          const void* scale_bf16, void* y, int y_is_f32, int B, int N, int K, int splits);

/* Self-test of the bounded-wait contract (the reference bounds its wait for the NPU by polling with a
 * timeout, runtime/torq_hw/src/TorqHw.cpp:172-186; here every wait INSIDE a kernel is bounded). Queues a
 * one-block kernel that waits, with the kernels' own wait helper and a limit of `limit_ms` (1..1000), on a
 * barrier that nothing completes. The kernel gives up, records code 99 and returns; the next tb200_wait()
 * therefore answers TB200_ABORTED once, and the device stays usable. */
int tb200_device_probe_bounded_wait(tb200_device_t* device, uint32_t limit_ms);

/* No counterpart in the reference (a measurement aid). Runs, on every SM of GPU `cuda_ordinal`,
 * `rounds` batches of 128 back-to-back tcgen05.mma kind::i8 instructions (M 128, N 256, K 32) on
 * operands resident in shared memory with TMEM accumulators - no memory traffic - and returns the
 * rate in tera-ops per second (1 multiply-accumulate = 2 ops) and the launch time. This is the
 * measured ceiling of the int8 tensor pipe that the contraction kernels' fractions are quoted
 * against. Synchronous; allocates a status word and a stream for its own use and frees them. */
int tb200_measure_i8_mma_peak(int cuda_ordinal, int rounds, double* tera_ops_per_s, double* ms);

/* No counterpart in the reference (a debugging aid). With TB200_GEMM_TRACE=1 in the environment, CTA 0 of every
 * tcgen05 GEMM / convolution launch records time stamps of its roles (6 roles x 512 slots: producer, MMA issuer,
 * four epilogue groups; each entry (nanoseconds << 8) | event tag, 0 = unused). This call waits for the current
 * device, copies up to `n` entries to `out`, clears the record and returns the count (-1 on failure). */
int tb200_debug_read_gemm_trace(unsigned long long* out, int n);

#ifdef __cplusplus
}
#endif
#endif /* TORQ_B200_H_ */
