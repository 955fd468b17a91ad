// Execution engine behind the C ABI of include/torq_b200.h: device, buffers,
// executable (parse + constant upload + launch plans + activation arena) and
// stream-ordered dispatch. It plays the part of runtime/driver/TorqExecutable.cc
// (initialize :655-752, executeDispatch :1025-1125) with the NPU action
// interpreter replaced by a list of CUDA launches. There is no CPU fallback:
// every failure surfaces as a status.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/torq_b200.h"
#include "../../include/torq_b200_ops.h"
#include "kernels.h"
#include "plan.h"
#include "tcgen05_ptx.cuh"

using namespace tb200;

struct tb200_device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;  // host-to-device uploads of the pipelined host call
  std::string last_error;
  std::mutex submit_mutex;  // one submission at a time, like the reference's
                            // per-executable mutex (TorqExecutable.cc:1043-1045)
  FILE* profile_csv = nullptr;
  uint64_t invocation_id = 0;
  int* status_word = nullptr;  // device word a kernel writes when one of its bounded waits expires
  int* status_host = nullptr;  // mapped pinned host word: the kernel that gives up stores its code here too (status_word.cuh)
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
};

struct tb200_buffer {
  tb200_device* dev = nullptr;
  void* ptr = nullptr;
  uint64_t bytes = 0;
  int memory_type = 0;
  bool owned = true;
};

namespace {

int fail(tb200_device* dev, int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (dev) dev->last_error = buf;
  return status;
}

#define CUDA_OK(dev, expr)                                                                   \
  do {                                                                                       \
    cudaError_t e_ = (expr);                                                                 \
    if (e_ != cudaSuccess)                                                                   \
      return fail(dev, e_ == cudaErrorMemoryAllocation ? TB200_RESOURCE_EXHAUSTED : TB200_INTERNAL, \
                  "%s failed: %s", #expr, cudaGetErrorString(e_));                          \
  } while (0)

size_t dtype_size(uint32_t d) {
  switch (d) {
    case TB200_I8: return 1;
    case TB200_I16: return 2;
    case TB200_BF16: return 2;
    case TB200_I32: return 4;
    case TB200_F32: return 4;
    case TB200_I64: return 8;
    default: return 0;
  }
}

uint64_t tensor_bytes(const tb200_tensor_t& t) {
  uint64_t n = dtype_size(t.dtype);
  for (uint32_t i = 0; i < 4; i++) n *= (uint64_t)(i < t.rank ? t.shape[i] : 1);
  return n;
}

}  // namespace

// ------------------------------------------------------------------ status / device

extern "C" const char* tb200_status_string(int s) {
  static const char* names[] = {"OK", "CANCELLED", "UNKNOWN", "INVALID_ARGUMENT", "DEADLINE_EXCEEDED",
                                "NOT_FOUND", "ALREADY_EXISTS", "PERMISSION_DENIED", "RESOURCE_EXHAUSTED",
                                "FAILED_PRECONDITION", "ABORTED", "OUT_OF_RANGE", "UNIMPLEMENTED",
                                "INTERNAL", "UNAVAILABLE", "DATA_LOSS"};
  if (s < 0 || s > 15) return "?";
  return names[s];
}

extern "C" int tb200_device_create(int ordinal, tb200_device_t** out) {
  if (!out) return TB200_INVALID_ARGUMENT;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) return TB200_UNAVAILABLE;  // no CPU fallback exists
  if (ordinal < 0 || ordinal >= count) return TB200_NOT_FOUND;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) return TB200_INTERNAL;
  if (prop.major != 10) return TB200_UNAVAILABLE;  // kernels are built for sm_100a only
  if (cudaSetDevice(ordinal) != cudaSuccess) return TB200_INTERNAL;
  auto* d = new tb200_device();
  d->ordinal = ordinal;
  if (cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete d;
    return TB200_INTERNAL;
  }
  if (cudaStreamCreateWithFlags(&d->copy_stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaStreamDestroy(d->stream);
    delete d;
    return TB200_INTERNAL;
  }
  int* mirror_dev = nullptr;
  if (cudaMalloc(&d->status_word, tb200::kStatusBlockBytes) != cudaSuccess ||
      cudaMemset(d->status_word, 0, tb200::kStatusBlockBytes) != cudaSuccess ||
      cudaHostAlloc((void**)&d->status_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess ||
      cudaHostGetDevicePointer((void**)&mirror_dev, d->status_host, 0) != cudaSuccess ||
      cudaMemcpy(reinterpret_cast<char*>(d->status_word) + 8, &mirror_dev, sizeof(mirror_dev), cudaMemcpyHostToDevice) !=
          cudaSuccess) {
    if (d->status_word) cudaFree(d->status_word);
    if (d->status_host) cudaFreeHost(d->status_host);
    cudaStreamDestroy(d->copy_stream);
    cudaStreamDestroy(d->stream);
    delete d;
    return TB200_RESOURCE_EXHAUSTED;
  }
  *d->status_host = 0;
  *out = d;
  return TB200_OK;
}

extern "C" int tb200_device_destroy(tb200_device_t* d) {
  if (!d) return TB200_INVALID_ARGUMENT;
  cudaSetDevice(d->ordinal);
  cudaStreamSynchronize(d->stream);
  cudaStreamSynchronize(d->copy_stream);
  cudaStreamDestroy(d->copy_stream);
  cudaStreamDestroy(d->stream);
  cudaFree(d->status_word);
  cudaFreeHost(d->status_host);
  if (d->profile_csv) fclose(d->profile_csv);
  delete d;
  return TB200_OK;
}

extern "C" int tb200_device_query_i64(tb200_device_t* d, const char* category, const char* key,
                                      int64_t* out) {
  if (!d || !category || !key || !out) return TB200_INVALID_ARGUMENT;
  *out = 0;
  if (!strcmp(category, "hal.executable.format")) {
    *out = !strcmp(key, TB200_OPS_FORMAT_STRING) ? 1 : 0;
    return TB200_OK;
  }
  if (!strcmp(category, "hal.device") || !strcmp(category, "hal.dispatch")) {
    if (!strcmp(key, "concurrency")) {
      *out = 1;
      return TB200_OK;
    }
  }
  return fail(d, TB200_NOT_FOUND, "unknown device configuration key value '%s :: %s'", category, key);
}

extern "C" void* tb200_device_stream(tb200_device_t* d) { return d ? (void*)d->stream : nullptr; }

extern "C" const char* tb200_last_error(tb200_device_t* d) { return d ? d->last_error.c_str() : ""; }

extern "C" int tb200_device_set_profile_csv(tb200_device_t* d, const char* path) {
  if (!d) return TB200_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  if (d->profile_csv) {
    fclose(d->profile_csv);
    d->profile_csv = nullptr;
  }
  if (path && *path) {
    d->profile_csv = fopen(path, "w");
    if (!d->profile_csv) return fail(d, TB200_PERMISSION_DENIED, "cannot open %s", path);
    fprintf(d->profile_csv, "dispatch_name,invocation_id,action_id,timestamp_us,event\n");
  }
  return TB200_OK;
}

// ------------------------------------------------------------------ buffers

namespace {
// With the host profiling log open, an explicit transfer is logged as a HOST_COPY event (the reference's
// name for host-side copies, runtime/torq_hw/inc/TorqEventLog.h:42) outside any dispatch: the first call
// (begin_us < 0) writes the _BEGIN row and returns its time, the second writes the _END row. The times are
// those of the enqueue: the copy itself is asynchronous.
long long profile_host_copy(tb200_device* d, long long begin_us) {
  if (!d->profile_csv) return 0;
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  if (!d->profile_csv) return 0;
  const long long t = (long long)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - d->t0).count();
  fprintf(d->profile_csv, "__HAL,%llu,-1,%lld,HOST_COPY_%s\n", (unsigned long long)d->invocation_id, begin_us < 0 ? t : std::max(t, begin_us),
          begin_us < 0 ? "BEGIN" : "END");
  return t;
}
}  // namespace

extern "C" int tb200_buffer_alloc(tb200_device_t* d, uint64_t bytes, int memory_type, tb200_buffer_t** out) {
  if (!d || !out) return TB200_INVALID_ARGUMENT;
  *out = nullptr;
  cudaSetDevice(d->ordinal);
  void* p = nullptr;
  uint64_t n = bytes ? bytes : 16;
  if (memory_type == TB200_MEMORY_DEVICE_LOCAL) {
    CUDA_OK(d, cudaMalloc(&p, n));
  } else if (memory_type == TB200_MEMORY_HOST_PINNED) {
    CUDA_OK(d, cudaHostAlloc(&p, n, cudaHostAllocDefault));
  } else {
    return fail(d, TB200_INVALID_ARGUMENT, "unknown memory type %d", memory_type);
  }
  auto* b = new tb200_buffer();
  b->dev = d;
  b->ptr = p;
  b->bytes = bytes;
  b->memory_type = memory_type;
  *out = b;
  return TB200_OK;
}

extern "C" int tb200_buffer_import(tb200_device_t* d, void* device_pointer, uint64_t bytes,
                                   tb200_buffer_t** out) {
  if (!d || !out || !device_pointer) return TB200_INVALID_ARGUMENT;
  auto* b = new tb200_buffer();
  b->dev = d;
  b->ptr = device_pointer;
  b->bytes = bytes;
  b->memory_type = TB200_MEMORY_DEVICE_LOCAL;
  b->owned = false;
  *out = b;
  return TB200_OK;
}

extern "C" int tb200_buffer_free(tb200_buffer_t* b) {
  if (!b) return TB200_INVALID_ARGUMENT;
  if (b->owned) {
    cudaSetDevice(b->dev->ordinal);
    cudaStreamSynchronize(b->dev->stream);
    if (b->memory_type == TB200_MEMORY_DEVICE_LOCAL) cudaFree(b->ptr);
    else cudaFreeHost(b->ptr);
  }
  delete b;
  return TB200_OK;
}

extern "C" int tb200_buffer_upload(tb200_buffer_t* b, uint64_t offset, const void* host, uint64_t bytes) {
  if (!b || (!host && bytes)) return TB200_INVALID_ARGUMENT;
  if (offset > b->bytes || bytes > b->bytes - offset) return fail(b->dev, TB200_OUT_OF_RANGE, "upload beyond end of buffer");
  cudaSetDevice(b->dev->ordinal);
  const long long t0 = profile_host_copy(b->dev, -1);
  CUDA_OK(b->dev, cudaMemcpyAsync((char*)b->ptr + offset, host, bytes, cudaMemcpyDefault, b->dev->stream));
  profile_host_copy(b->dev, t0);
  return TB200_OK;
}

extern "C" int tb200_buffer_download(tb200_buffer_t* b, uint64_t offset, void* host, uint64_t bytes) {
  if (!b || (!host && bytes)) return TB200_INVALID_ARGUMENT;
  if (offset > b->bytes || bytes > b->bytes - offset) return fail(b->dev, TB200_OUT_OF_RANGE, "download beyond end of buffer");
  cudaSetDevice(b->dev->ordinal);
  const long long t0 = profile_host_copy(b->dev, -1);
  CUDA_OK(b->dev, cudaMemcpyAsync(host, (const char*)b->ptr + offset, bytes, cudaMemcpyDefault, b->dev->stream));
  profile_host_copy(b->dev, t0);
  return TB200_OK;
}

extern "C" void* tb200_buffer_pointer(tb200_buffer_t* b) { return b ? b->ptr : nullptr; }
extern "C" uint64_t tb200_buffer_size(tb200_buffer_t* b) { return b ? b->bytes : 0; }

// ------------------------------------------------------------------ executable

struct tb200_executable {
  tb200_device* dev = nullptr;
  std::vector<tb200_tensor_t> tensors;
  std::vector<tb200_op_t> ops;
  std::vector<int32_t> inputs, outputs;
  std::vector<uint8_t> constants;  // host copy of the constants section
  Plan plan;                       // launch list + arena layout (plan.h)
  void* arena = nullptr;
  void* const_dev = nullptr;       // derived constants (packed weights, channel params)
  // tb200_invoke_host[_async]: two sets of device staging buffers, used alternately, so the
  // upload of one call overlaps the kernels of the previous one
  std::vector<tb200_buffer_t*> staging_in[2], staging_out[2];
  cudaEvent_t ev_uploaded[2] = {nullptr, nullptr}, ev_released[2] = {nullptr, nullptr};
  uint64_t host_calls = 0;
  // CUDA graphs of the whole launch list, one per distinct set of bound addresses
  // (a dispatch with the same bindings replays its graph: one submission instead of
  // one per kernel). Small LRU; TB200_NO_GRAPH=1 turns it off.
  struct CachedGraph {
    std::vector<void*> io;
    cudaGraphExec_t exec = nullptr;
    uint64_t last_use = 0;
  };
  std::vector<CachedGraph> graphs;
  uint64_t graph_clock = 0;
  // tensor parallelism: the scratch area of every member of the group as mapped into this
  // process (own entry = own scratch); mapped[r] = base of a peer's arena opened through IPC
  char* peer_scratch[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  void* peer_mapped[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  bool peers_connected = false;
};

extern "C" int tb200_executable_create(tb200_device_t* d, const void* bytes, size_t n_bytes,
                                       tb200_executable_t** out) {
  if (!d || !bytes || !out) return TB200_INVALID_ARGUMENT;
  *out = nullptr;
  if (n_bytes < sizeof(tb200_ops_header_t)) return fail(d, TB200_INVALID_ARGUMENT, "blob shorter than its header");
  tb200_ops_header_t h;
  memcpy(&h, bytes, sizeof(h));
  // a blob of another format: NOT_FOUND, as the reference's executable cache answers for a format it has
  // no implementation for (runtime/driver/nop_executable_cache.cc:97-105)
  if (h.magic != TB200_OPS_MAGIC)
    return fail(d, TB200_NOT_FOUND, "no executable implementation for this format: not a %s blob (bad magic)",
                TB200_OPS_FORMAT_STRING);
  if (h.version != TB200_OPS_VERSION)
    return fail(d, TB200_UNAVAILABLE, "executable version %u is not compatible with runtime version %u",
                h.version, TB200_OPS_VERSION);
  if (h.total_bytes > n_bytes) return fail(d, TB200_INVALID_ARGUMENT, "blob truncated: %llu > %zu",
                                           (unsigned long long)h.total_bytes, n_bytes);
  auto in_range = [&](uint64_t off, uint64_t len) { return off <= n_bytes && len <= n_bytes - off; };
  if (!in_range(h.tensors_offset, (uint64_t)h.n_tensors * sizeof(tb200_tensor_t)) ||
      !in_range(h.ops_offset, (uint64_t)h.n_ops * sizeof(tb200_op_t)) ||
      !in_range(h.inputs_offset, (uint64_t)h.n_inputs * 4) ||
      !in_range(h.outputs_offset, (uint64_t)h.n_outputs * 4) || !in_range(h.const_offset, h.const_bytes))
    return fail(d, TB200_INVALID_ARGUMENT, "section outside the blob");

  auto* ex = new tb200_executable();
  ex->dev = d;
  const char* base = (const char*)bytes;
  ex->tensors.resize(h.n_tensors);
  memcpy(ex->tensors.data(), base + h.tensors_offset, h.n_tensors * sizeof(tb200_tensor_t));
  ex->ops.resize(h.n_ops);
  memcpy(ex->ops.data(), base + h.ops_offset, h.n_ops * sizeof(tb200_op_t));
  ex->inputs.resize(h.n_inputs);
  memcpy(ex->inputs.data(), base + h.inputs_offset, h.n_inputs * 4);
  ex->outputs.resize(h.n_outputs);
  memcpy(ex->outputs.data(), base + h.outputs_offset, h.n_outputs * 4);
  ex->constants.assign(base + h.const_offset, base + h.const_offset + h.const_bytes);

  std::string err;
  int st = TB200_OK;
  for (size_t i = 0; i < ex->tensors.size() && st == TB200_OK; i++) {
    const auto& t = ex->tensors[i];
    if (t.rank < 1 || t.rank > 4 || dtype_size(t.dtype) == 0) st = fail(d, TB200_INVALID_ARGUMENT, "tensor %zu: bad rank/dtype", i);
    for (uint32_t k = 0; k < t.rank && st == TB200_OK; k++)
      if (t.shape[k] <= 0) st = fail(d, TB200_INVALID_ARGUMENT, "tensor %zu: non-positive extent", i);
    if (st == TB200_OK && t.kind == TB200_TENSOR_CONSTANT &&
        (t.const_offset > h.const_bytes || t.const_bytes > h.const_bytes - t.const_offset ||
         t.const_bytes < tensor_bytes(t)))
      st = fail(d, TB200_INVALID_ARGUMENT, "tensor %zu: constant outside the constants section", i);
  }
  for (int32_t id : ex->inputs)
    if (st == TB200_OK && (id < 0 || id >= (int)h.n_tensors || ex->tensors[id].kind != TB200_TENSOR_INPUT))
      st = fail(d, TB200_INVALID_ARGUMENT, "input list names tensor %d which is not an input", id);
  for (int32_t id : ex->outputs)
    if (st == TB200_OK && (id < 0 || id >= (int)h.n_tensors || ex->tensors[id].kind != TB200_TENSOR_OUTPUT))
      st = fail(d, TB200_INVALID_ARGUMENT, "output list names tensor %d which is not an output", id);
  if (st != TB200_OK) {
    delete ex;
    return st;
  }

  // io slot of a bound tensor = its position among inputs, then outputs
  for (size_t i = 0; i < ex->inputs.size(); i++) ex->tensors[ex->inputs[i]].reserved = (uint32_t)i;
  for (size_t i = 0; i < ex->outputs.size(); i++)
    ex->tensors[ex->outputs[i]].reserved = (uint32_t)(ex->inputs.size() + i);
  cudaSetDevice(d->ordinal);
  st = build_plan(ex->tensors, ex->ops, ex->constants, ex->plan, err);
  if (st != TB200_OK) {
    fail(d, st, "%s", err.c_str());
    delete ex;
    return st;
  }
  // device memory: activation arena + derived constants, one allocation each
  cudaError_t e = cudaSuccess;
  if (ex->plan.arena_bytes) e = cudaMalloc(&ex->arena, ex->plan.arena_bytes);
  if (e == cudaSuccess && !ex->plan.const_image.empty()) {
    e = cudaMalloc(&ex->const_dev, ex->plan.const_image.size());
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(ex->const_dev, ex->plan.const_image.data(), ex->plan.const_image.size(),
                          cudaMemcpyHostToDevice, d->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
  }
  if (e == cudaSuccess && ex->plan.state_bytes) {
    // persistent state tensors live at the front of the arena and start at zero
    e = cudaMemsetAsync(ex->arena, 0, ex->plan.state_bytes, d->stream);
  }
  if (e == cudaSuccess && ex->plan.zero_scratch && ex->plan.scratch_bytes)
    e = cudaMemsetAsync((char*)ex->arena + ex->plan.scratch_offset, 0, ex->plan.scratch_bytes, d->stream);
  if (e != cudaSuccess) {
    st = fail(d, e == cudaErrorMemoryAllocation ? TB200_RESOURCE_EXHAUSTED : TB200_INTERNAL,
              "executable memory: %s", cudaGetErrorString(e));
    if (ex->arena) cudaFree(ex->arena);
    if (ex->const_dev) cudaFree(ex->const_dev);
    delete ex;
    return st;
  }
  *out = ex;
  return TB200_OK;
}

extern "C" int tb200_executable_destroy(tb200_executable_t* ex) {
  if (!ex) return TB200_INVALID_ARGUMENT;
  cudaSetDevice(ex->dev->ordinal);
  cudaStreamSynchronize(ex->dev->stream);
  for (auto& g : ex->graphs) cudaGraphExecDestroy(g.exec);
  cudaStreamSynchronize(ex->dev->copy_stream);
  for (int s = 0; s < 2; s++) {
    for (auto* b : ex->staging_in[s]) tb200_buffer_free(b);
    for (auto* b : ex->staging_out[s]) tb200_buffer_free(b);
    if (ex->ev_uploaded[s]) cudaEventDestroy(ex->ev_uploaded[s]);
    if (ex->ev_released[s]) cudaEventDestroy(ex->ev_released[s]);
  }
  for (void* m : ex->peer_mapped)
    if (m) cudaIpcCloseMemHandle(m);
  if (ex->arena) cudaFree(ex->arena);
  if (ex->const_dev) cudaFree(ex->const_dev);
  delete ex;
  return TB200_OK;
}

// ---- tensor-parallel groups: one process per GPU; the members exchange handles out of band ----
namespace {
struct CommHandle {  // the 96 bytes of tb200_comm_handle_t
  cudaIpcMemHandle_t mem;  // the executable's arena allocation
  uint64_t scratch_offset;
  int32_t rank, tp;
  uint8_t pad[16];
};
static_assert(sizeof(CommHandle) == sizeof(tb200_comm_handle_t), "tb200_comm_handle_t size");
}  // namespace

extern "C" int tb200_executable_comm_info(tb200_executable_t* ex, int32_t* rank, int32_t* group_size) {
  if (!ex || !rank || !group_size) return TB200_INVALID_ARGUMENT;
  *rank = ex->plan.rank;
  *group_size = ex->plan.tp;
  return TB200_OK;
}

extern "C" int tb200_executable_comm_handle(tb200_executable_t* ex, tb200_comm_handle_t* out) {
  if (!ex || !out) return TB200_INVALID_ARGUMENT;
  tb200_device* d = ex->dev;
  if (ex->plan.tp < 2) return fail(d, TB200_FAILED_PRECONDITION, "the executable is not a tensor-parallel shard");
  cudaSetDevice(d->ordinal);
  CommHandle h{};
  CUDA_OK(d, cudaIpcGetMemHandle(&h.mem, ex->arena));
  h.scratch_offset = ex->plan.scratch_offset;
  h.rank = ex->plan.rank;
  h.tp = ex->plan.tp;
  memcpy(out, &h, sizeof(h));
  return TB200_OK;
}

extern "C" int tb200_executable_connect_peers(tb200_executable_t* ex, const tb200_comm_handle_t* handles, size_t n) {
  if (!ex || !handles) return TB200_INVALID_ARGUMENT;
  tb200_device* d = ex->dev;
  const int tp = ex->plan.tp, rank = ex->plan.rank;
  if (tp < 2) return fail(d, TB200_FAILED_PRECONDITION, "the executable is not a tensor-parallel shard");
  if ((int)n != tp) return fail(d, TB200_INVALID_ARGUMENT, "%zu handles for a group of %d", n, tp);
  if (ex->peers_connected) return fail(d, TB200_FAILED_PRECONDITION, "the peers are already connected");
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  cudaSetDevice(d->ordinal);
  for (int r = 0; r < tp; r++) {
    CommHandle h;
    memcpy(&h, &handles[r], sizeof(h));
    if (h.rank != r || h.tp != tp)
      return fail(d, TB200_INVALID_ARGUMENT, "handle %d describes rank %d of a group of %d", r, h.rank, h.tp);
    if (r == rank) {
      ex->peer_scratch[r] = (char*)ex->arena + ex->plan.scratch_offset;
      continue;
    }
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h.mem, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return fail(d, TB200_UNAVAILABLE, "cannot map rank %d's memory (peer access over NVLink/PCIe needed): %s", r,
                  cudaGetErrorString(e));
    ex->peer_mapped[r] = base;
    ex->peer_scratch[r] = (char*)base + h.scratch_offset;
  }
  ex->peers_connected = true;
  return TB200_OK;
}

extern "C" int tb200_executable_io_count(tb200_executable_t* ex, uint32_t* n_in, uint32_t* n_out) {
  if (!ex) return TB200_INVALID_ARGUMENT;
  if (n_in) *n_in = (uint32_t)ex->inputs.size();
  if (n_out) *n_out = (uint32_t)ex->outputs.size();
  return TB200_OK;
}

extern "C" int tb200_executable_io_info(tb200_executable_t* ex, int is_output, uint32_t index,
                                        tb200_io_info_t* info) {
  if (!ex || !info) return TB200_INVALID_ARGUMENT;
  const auto& ids = is_output ? ex->outputs : ex->inputs;
  if (index >= ids.size()) return fail(ex->dev, TB200_OUT_OF_RANGE, "io index %u out of range", index);
  const auto& t = ex->tensors[ids[index]];
  info->dtype = t.dtype;
  info->rank = t.rank;
  for (int i = 0; i < 4; i++) info->shape[i] = (uint32_t)i < t.rank ? t.shape[i] : 1;
  info->bytes = tensor_bytes(t);
  return TB200_OK;
}

extern "C" uint32_t tb200_executable_op_count(tb200_executable_t* ex) { return ex ? (uint32_t)ex->ops.size() : 0; }
extern "C" uint32_t tb200_executable_launch_count(tb200_executable_t* ex) {
  return ex ? (uint32_t)ex->plan.launch_count : 0;
}
extern "C" const char* tb200_executable_op_kernel(tb200_executable_t* ex, uint32_t index) {
  if (!ex || index >= ex->plan.steps.size()) return "";
  return ex->plan.steps[index].kernel_name;
}

namespace {

// Resolve the binding list (inputs then outputs) to device addresses, with the
// checks of torq_command_buffer.c:488-495 and TorqExecutable.cc:512-531.
int resolve_bindings(tb200_executable* ex, const tb200_binding_t* bindings, size_t n, std::vector<void*>& io) {
  tb200_device* d = ex->dev;
  size_t want = ex->inputs.size() + ex->outputs.size();
  if (n != want) return fail(d, TB200_INVALID_ARGUMENT, "expected %zu bindings, got %zu", want, n);
  if (n && !bindings) return TB200_INVALID_ARGUMENT;
  io.resize(n);
  for (size_t i = 0; i < n; i++) {
    const auto& b = bindings[i];
    // runtime/driver/torq_command_buffer.c:488-495: a NULL binding is FAILED_PRECONDITION
    if (!b.buffer || !b.buffer->ptr)
      return fail(d, TB200_FAILED_PRECONDITION, "required binding %zu is NULL; all bindings must have a valid pointer", i);
    int32_t tid = i < ex->inputs.size() ? ex->inputs[i] : ex->outputs[i - ex->inputs.size()];
    uint64_t need = tensor_bytes(ex->tensors[tid]);
    if (b.offset > b.buffer->bytes) return fail(d, TB200_OUT_OF_RANGE, "binding %zu offset beyond buffer", i);
    uint64_t len = b.length ? b.length : b.buffer->bytes - b.offset;
    if (len > b.buffer->bytes - b.offset || len < need)
      return fail(d, TB200_OUT_OF_RANGE, "binding %zu: %llu bytes bound, tensor needs %llu", i,
                  (unsigned long long)len, (unsigned long long)need);
    // the kernels use 16-byte vector accesses and TMA on bound tensors: the bound ADDRESS must be aligned
    if (((uintptr_t)b.buffer->ptr + b.offset) & 15)
      return fail(d, TB200_INVALID_ARGUMENT, "binding %zu: address (buffer + offset) must be 16-byte aligned", i);
    if (b.buffer->memory_type != TB200_MEMORY_DEVICE_LOCAL)
      return fail(d, TB200_FAILED_PRECONDITION, "binding %zu is not device-local memory", i);
    io[i] = (char*)b.buffer->ptr + b.offset;
  }
  return TB200_OK;
}

long long now_us(tb200_device* d) {
  return (long long)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - d->t0).count();
}

// One row of the host profiling log. Columns, event names and the _BEGIN/_END suffixes are the
// reference's (runtime/torq_hw/src/TorqEventLog.cpp:49,95-100; names runtime/torq_hw/inc/TorqEventLog.h:19-49);
// timestamps are whole microseconds like its, so its readers (python/torq/debug_info.py:84) parse the file.
void csv_row(tb200_device* d, const char* name, uint64_t invocation, long long action, long long t_us, const char* event,
             bool begin) {
  fprintf(d->profile_csv, "%s,%llu,%lld,%lld,%s_%s\n", name, (unsigned long long)invocation, action, t_us, event,
          begin ? "BEGIN" : "END");
}

int run_plan(tb200_executable* ex, const std::vector<void*>& io, std::vector<cudaEvent_t>* events) {
  tb200_device* d = ex->dev;
  ExecContext ctx;
  ctx.arena = (char*)ex->arena;
  ctx.consts = (char*)ex->const_dev;
  ctx.io = io.data();
  ctx.stream = d->stream;
  ctx.status = d->status_word;
  ctx.scratch = (char*)ex->arena + ex->plan.scratch_offset;
  cudaError_t launch_error = cudaSuccess;
  ctx.launch_error = &launch_error;
  ctx.peer_scratch = ex->peers_connected ? ex->peer_scratch : nullptr;
  for (size_t i = 0; i < ex->plan.steps.size(); i++) {
    if (events) cudaEventRecord((*events)[i], d->stream);
    ex->plan.steps[i].launch(ctx);
  }
  if (events) cudaEventRecord((*events)[ex->plan.steps.size()], d->stream);
  CUDA_OK(d, launch_error);
  CUDA_OK(d, cudaGetLastError());
  return TB200_OK;
}

bool use_graphs() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("TB200_NO_GRAPH");
    v = (e && *e && *e != '0') ? 0 : 1;
  }
  return v == 1;
}

// Replays (or first captures) the CUDA graph of the launch list for this set of addresses.
int run_graph(tb200_executable* ex, const std::vector<void*>& io) {
  tb200_device* d = ex->dev;
  constexpr size_t kMaxGraphs = 8;
  ex->graph_clock++;
  for (auto& g : ex->graphs)
    if (g.io == io) {
      g.last_use = ex->graph_clock;
      CUDA_OK(d, cudaGraphLaunch(g.exec, d->stream));
      return TB200_OK;
    }
  // tensor maps and function attributes are set up by a first direct run, outside any capture
  int st = run_plan(ex, io, nullptr);
  if (st != TB200_OK) return st;
  cudaGraph_t graph = nullptr;
  CUDA_OK(d, cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
  st = run_plan(ex, io, nullptr);
  cudaError_t e = cudaStreamEndCapture(d->stream, &graph);
  if (st != TB200_OK || e != cudaSuccess) {
    if (graph) cudaGraphDestroy(graph);
    return st != TB200_OK ? st : fail(d, TB200_INTERNAL, "graph capture failed: %s", cudaGetErrorString(e));
  }
  tb200_executable::CachedGraph cg;
  cg.io = io;
  cg.last_use = ex->graph_clock;
  e = cudaGraphInstantiate(&cg.exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(d, TB200_INTERNAL, "graph instantiate failed: %s", cudaGetErrorString(e));
  if (ex->graphs.size() >= kMaxGraphs) {
    size_t victim = 0;
    for (size_t i = 1; i < ex->graphs.size(); i++)
      if (ex->graphs[i].last_use < ex->graphs[victim].last_use) victim = i;
    cudaGraphExecDestroy(ex->graphs[victim].exec);
    ex->graphs.erase(ex->graphs.begin() + victim);
  }
  ex->graphs.push_back(cg);
  // the direct run above already produced this dispatch's results
  return TB200_OK;
}

// Host-side copies that bracket a profiled dispatch (tb200_invoke_host): run inside the
// DISPATCH_SYNC_BINDINGS_IN / _OUT events, like the reference's binding syncs
// (runtime/driver/TorqExecutable.cc:1071-1073,1088-1090).
struct HostSync {
  std::function<int()> copy_in, copy_out;
};

// The dispatch proper; the caller holds submit_mutex and has made the device current.
int dispatch_locked(tb200_executable* ex, const std::vector<void*>& io, const HostSync* host) {
  tb200_device* d = ex->dev;
  if (!d->profile_csv) {
    int st = TB200_OK;
    if (host && host->copy_in && (st = host->copy_in()) != TB200_OK) return st;
    st = use_graphs() && ex->plan.use_graph ? run_graph(ex, io) : run_plan(ex, io, nullptr);
    if (st == TB200_OK && host && host->copy_out) st = host->copy_out();
    return st;
  }
  // Profiled dispatch: synchronous, every op bracketed by CUDA events. An op's kernel plays the part of an
  // NSS job of the reference: its NSS_START_BEGIN / NSS_START_END rows bracket the device execution.
  const size_t ns = ex->plan.steps.size();
  std::vector<cudaEvent_t> ev(ns + 1);
  for (auto& e : ev) cudaEventCreate(&e);
  const uint64_t inv = d->invocation_id++;
  const char* name = "dispatch";
  int st = TB200_OK;
  csv_row(d, name, inv, -1, now_us(d), "DISPATCH", true);
  csv_row(d, name, inv, -1, now_us(d), "DISPATCH_SYNC_BINDINGS_IN", true);
  if (host && host->copy_in) st = host->copy_in();
  if (st == TB200_OK && cudaStreamSynchronize(d->stream) != cudaSuccess) st = fail(d, TB200_INTERNAL, "stream failed before the dispatch");
  csv_row(d, name, inv, -1, now_us(d), "DISPATCH_SYNC_BINDINGS_IN", false);
  if (st == TB200_OK) {
    const long long t_begin = now_us(d);
    csv_row(d, name, inv, -1, t_begin, "DISPATCH_EXECUTE_ACTIONS", true);
    st = run_plan(ex, io, &ev);
    if (st == TB200_OK && cudaStreamSynchronize(d->stream) != cudaSuccess) st = fail(d, TB200_INTERNAL, "stream failed in the dispatch");
    long long t_last = t_begin;
    if (st == TB200_OK) {
      // device times of the ops, placed after the host time at which the launches began
      double acc_us = 0.0;
      for (size_t i = 0; i < ns; i++) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
        const long long b = t_begin + (long long)(acc_us + 0.5);
        acc_us += (double)ms * 1e3;
        const long long e = t_begin + (long long)(acc_us + 0.5);
        if (ex->plan.steps[i].launches == 0) continue;  // views and ops fused into a neighbour launch nothing
        csv_row(d, ex->plan.steps[i].kernel_name, inv, (long long)i, b, "NSS_START", true);
        csv_row(d, ex->plan.steps[i].kernel_name, inv, (long long)i, e, "NSS_START", false);
        t_last = e;
      }
    }
    const long long t_end = std::max(now_us(d), t_last);
    csv_row(d, name, inv, -1, t_end, "DISPATCH_EXECUTE_ACTIONS", false);
    csv_row(d, name, inv, -1, t_end, "DISPATCH_SYNC_BINDINGS_OUT", true);
    if (st == TB200_OK && host && host->copy_out) {
      st = host->copy_out();
      if (st == TB200_OK && cudaStreamSynchronize(d->stream) != cudaSuccess) st = fail(d, TB200_INTERNAL, "stream failed after the dispatch");
    }
    csv_row(d, name, inv, -1, std::max(now_us(d), t_end), "DISPATCH_SYNC_BINDINGS_OUT", false);
  }
  csv_row(d, name, inv, -1, std::max(now_us(d), (long long)0), "DISPATCH", false);
  fflush(d->profile_csv);
  for (auto& e : ev) cudaEventDestroy(e);
  return st;
}

}  // namespace

extern "C" int tb200_dispatch(tb200_executable_t* ex, const tb200_binding_t* bindings, size_t n) {
  if (!ex) return TB200_INVALID_ARGUMENT;
  tb200_device* d = ex->dev;
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  cudaSetDevice(d->ordinal);
  std::vector<void*> io;
  int st = resolve_bindings(ex, bindings, n, io);
  if (st != TB200_OK) return st;
  return dispatch_locked(ex, io, nullptr);
}

extern "C" int tb200_wait(tb200_device_t* d, uint64_t timeout_ns) {
  if (!d) return TB200_INVALID_ARGUMENT;
  cudaSetDevice(d->ordinal);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
  for (;;) {
    cudaError_t e = cudaStreamQuery(d->stream);
    if (e == cudaSuccess) {
      // The stream drained: did a kernel give up on one of its bounded waits? The kernel that gives up stores
      // its code in this mapped host word as well as in the device word, so this is a plain read.
      const int code = *(volatile int*)d->status_host;
      if (code != 0) {
        *(volatile int*)d->status_host = 0;
        cudaMemsetAsync(d->status_word, 0, sizeof(int), d->stream);
        return fail(d, TB200_ABORTED, "a kernel's bounded wait expired (code %d); results of this dispatch are invalid", code);
      }
      return TB200_OK;
    }
    if (e != cudaErrorNotReady) return fail(d, TB200_INTERNAL, "stream failed: %s", cudaGetErrorString(e));
    if (std::chrono::steady_clock::now() >= deadline)
      return fail(d, TB200_DEADLINE_EXCEEDED, "device did not finish within %llu ns", (unsigned long long)timeout_ns);
  }
}

namespace {
// Frees whatever a failed set-up of the host-call staging left behind, so the next call starts over.
void drop_staging(tb200_executable* ex) {
  for (int s = 0; s < 2; s++) {
    for (auto* b : ex->staging_in[s]) tb200_buffer_free(b);
    for (auto* b : ex->staging_out[s]) tb200_buffer_free(b);
    ex->staging_in[s].clear();
    ex->staging_out[s].clear();
    if (ex->ev_uploaded[s]) cudaEventDestroy(ex->ev_uploaded[s]);
    if (ex->ev_released[s]) cudaEventDestroy(ex->ev_released[s]);
    ex->ev_uploaded[s] = ex->ev_released[s] = nullptr;
  }
}
}  // namespace

extern "C" int tb200_invoke_host_async(tb200_executable_t* ex, const void* const* host_inputs,
                                       void* const* host_outputs) {
  if (!ex || (!host_inputs && !ex->inputs.empty()) || (!host_outputs && !ex->outputs.empty()))
    return TB200_INVALID_ARGUMENT;
  tb200_device* d = ex->dev;
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  cudaSetDevice(d->ordinal);
  const size_t ni = ex->inputs.size(), no = ex->outputs.size();
  for (size_t i = 0; i < ni; i++)
    if (!host_inputs[i]) return fail(d, TB200_FAILED_PRECONDITION, "host input %zu is NULL; all bindings must have a valid pointer", i);
  for (size_t i = 0; i < no; i++)
    if (!host_outputs[i]) return fail(d, TB200_FAILED_PRECONDITION, "host output %zu is NULL; all bindings must have a valid pointer", i);
  if (!ex->ev_uploaded[1]) {
    drop_staging(ex);  // nothing, or the remains of a set-up that failed half way
    int st = TB200_OK;
    for (int s = 0; s < 2 && st == TB200_OK; s++) {
      for (size_t i = 0; i < ni && st == TB200_OK; i++) {
        tb200_buffer_t* b = nullptr;
        st = tb200_buffer_alloc(d, tensor_bytes(ex->tensors[ex->inputs[i]]), TB200_MEMORY_DEVICE_LOCAL, &b);
        if (st == TB200_OK) ex->staging_in[s].push_back(b);
      }
      for (size_t i = 0; i < no && st == TB200_OK; i++) {
        tb200_buffer_t* b = nullptr;
        st = tb200_buffer_alloc(d, tensor_bytes(ex->tensors[ex->outputs[i]]), TB200_MEMORY_DEVICE_LOCAL, &b);
        if (st == TB200_OK) ex->staging_out[s].push_back(b);
      }
      if (st == TB200_OK && cudaEventCreateWithFlags(&ex->ev_released[s], cudaEventDisableTiming) != cudaSuccess)
        st = fail(d, TB200_INTERNAL, "cannot create an event");
      if (st == TB200_OK && cudaEventCreateWithFlags(&ex->ev_uploaded[s], cudaEventDisableTiming) != cudaSuccess)
        st = fail(d, TB200_INTERNAL, "cannot create an event");
    }
    if (st != TB200_OK) {
      drop_staging(ex);
      return st;
    }
  }
  const int s = (int)(ex->host_calls & 1);
  const bool reused = ex->host_calls >= 2;
  ex->host_calls++;
  std::vector<void*> io(ni + no);
  for (size_t i = 0; i < ni; i++) io[i] = ex->staging_in[s][i]->ptr;
  for (size_t i = 0; i < no; i++) io[ni + i] = ex->staging_out[s][i]->ptr;
  HostSync host;
  host.copy_in = [&]() -> int {
    // upload stream: wait until the call two back has released this staging set, then copy in
    if (reused) CUDA_OK(d, cudaStreamWaitEvent(d->copy_stream, ex->ev_released[s], 0));
    for (size_t i = 0; i < ni; i++)
      CUDA_OK(d, cudaMemcpyAsync(ex->staging_in[s][i]->ptr, host_inputs[i], ex->staging_in[s][i]->bytes,
                                 cudaMemcpyHostToDevice, d->copy_stream));
    CUDA_OK(d, cudaEventRecord(ex->ev_uploaded[s], d->copy_stream));
    // compute stream: wait for the upload
    CUDA_OK(d, cudaStreamWaitEvent(d->stream, ex->ev_uploaded[s], 0));
    return TB200_OK;
  };
  host.copy_out = [&]() -> int {
    for (size_t i = 0; i < no; i++)
      CUDA_OK(d, cudaMemcpyAsync(host_outputs[i], ex->staging_out[s][i]->ptr, ex->staging_out[s][i]->bytes,
                                 cudaMemcpyDeviceToHost, d->stream));
    CUDA_OK(d, cudaEventRecord(ex->ev_released[s], d->stream));
    return TB200_OK;
  };
  return dispatch_locked(ex, io, &host);
}

namespace {
// A wait that nothing ever completes, bounded like every wait of the real kernels (same helper).
__global__ void wait_probe_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    tb200::mbar_init(tb200::smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) tb200::mbar_wait(tb200::smem_u32(&bar), 0, status, 99, limit_ns);
}
}  // namespace

extern "C" int tb200_device_probe_bounded_wait(tb200_device_t* d, uint32_t limit_ms) {
  if (!d || limit_ms < 1 || limit_ms > 1000) return TB200_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  cudaSetDevice(d->ordinal);
  wait_probe_kernel<<<1, 32, 0, d->stream>>>(d->status_word, (unsigned long long)limit_ms * 1000000ull);
  CUDA_OK(d, cudaGetLastError());
  return TB200_OK;
}

extern "C" int tb200_debug_read_gemm_trace(unsigned long long* out, int n) {
  if (!out || n <= 0) return -1;
  return tb200::read_gemm_trace(out, n);
}

extern "C" int tb200_invoke_host(tb200_executable_t* ex, const void* const* host_inputs,
                                 void* const* host_outputs) {
  int st = tb200_invoke_host_async(ex, host_inputs, host_outputs);
  if (st != TB200_OK) return st;
  CUDA_OK(ex->dev, cudaStreamSynchronize(ex->dev->stream));
  return TB200_OK;
}

extern "C" int tb200_executable_profile_ops(tb200_executable_t* ex, const tb200_binding_t* bindings,
                                            size_t n, int warmup, int iters, float* ms, uint32_t cap) {
  if (!ex || !ms || iters <= 0) return TB200_INVALID_ARGUMENT;
  tb200_device* d = ex->dev;
  size_t ns = ex->plan.steps.size();
  if (cap < ns) return fail(d, TB200_OUT_OF_RANGE, "ms array holds %u entries, executable has %zu ops", cap, ns);
  std::lock_guard<std::mutex> lock(d->submit_mutex);
  cudaSetDevice(d->ordinal);
  std::vector<void*> io;
  int st = resolve_bindings(ex, bindings, n, io);
  if (st != TB200_OK) return st;
  for (int i = 0; i < warmup; i++)
    if ((st = run_plan(ex, io, nullptr)) != TB200_OK) return st;
  std::vector<cudaEvent_t> ev(ns + 1);
  for (auto& e : ev) cudaEventCreate(&e);
  for (size_t i = 0; i < ns; i++) ms[i] = 0.f;
  for (int it = 0; it < iters && st == TB200_OK; it++) {
    st = run_plan(ex, io, &ev);
    if (st != TB200_OK) break;
    cudaStreamSynchronize(d->stream);
    for (size_t i = 0; i < ns; i++) {
      float t = 0.f;
      cudaEventElapsedTime(&t, ev[i], ev[i + 1]);
      ms[i] += t / iters;
    }
  }
  for (auto& e : ev) cudaEventDestroy(e);
  return st;
}
