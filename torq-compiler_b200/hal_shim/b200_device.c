// iree_hal_device_t of the torq_b200 HAL driver: one CUDA device behind the C ABI. The 31 slots are those of
// runtime/driver/torq_device.c:570-602 of the reference. Queue operations follow the reference's shape
// (wait semaphores -> apply -> signal, torq_device.c:487-526) and stay synchronous at this surface: the
// device's stream is drained (tb200_wait) before the signal, so a signalled semaphore means finished work.
// Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"
#include "iree/hal/utils/deferred_command_buffer.h"
#include "iree/hal/utils/file_registry.h"
#include "iree/hal/utils/file_transfer.h"
#include "iree/hal/utils/queue_emulation.h"

typedef struct b200_device_t {
  iree_hal_resource_t resource;
  iree_string_view_t identifier;  // storage follows the struct
  iree_allocator_t host_allocator;
  iree_hal_allocator_t* device_allocator;
  iree_arena_block_pool_t block_pool;  // deferred command buffers record into it
  tb200_device_t* handle;
  int cuda_ordinal;
} b200_device_t;

static const iree_hal_device_vtable_t b200_device_vtable;

static b200_device_t* b200_device_cast(iree_hal_device_t* base) {
  IREE_HAL_ASSERT_TYPE(base, &b200_device_vtable);
  return (b200_device_t*)base;
}

tb200_device_t* iree_hal_torq_b200_device_handle(iree_hal_device_t* device) { return b200_device_cast(device)->handle; }

iree_status_t iree_hal_torq_b200_device_create(iree_string_view_t identifier, int cuda_ordinal,
                                               iree_allocator_t host_allocator, iree_hal_device_t** out_device) {
  *out_device = NULL;
  b200_device_t* device = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, sizeof(*device) + identifier.size, (void**)&device));
  memset(device, 0, sizeof(*device));
  iree_hal_resource_initialize(&b200_device_vtable, &device->resource);
  iree_string_view_append_to_buffer(identifier, &device->identifier, (char*)device + sizeof(*device));
  device->host_allocator = host_allocator;
  device->cuda_ordinal = cuda_ordinal;
  iree_arena_block_pool_initialize(32 * 1024, host_allocator, &device->block_pool);
  // UNAVAILABLE when there is no sm_100 GPU: this driver has no other way to execute
  iree_status_t status = iree_hal_torq_b200_status(tb200_device_create(cuda_ordinal, &device->handle), NULL, "tb200_device_create");
  if (iree_status_is_ok(status)) {
    status = iree_hal_torq_b200_allocator_create(device->handle, host_allocator, &device->device_allocator);
  }
  if (iree_status_is_ok(status)) {
    *out_device = (iree_hal_device_t*)device;
  } else {
    iree_hal_device_release((iree_hal_device_t*)device);
  }
  return status;
}

static void b200_device_destroy(iree_hal_device_t* base) {
  b200_device_t* device = b200_device_cast(base);
  iree_hal_allocator_release(device->device_allocator);
  if (device->handle) tb200_device_destroy(device->handle);
  iree_arena_block_pool_deinitialize(&device->block_pool);
  iree_allocator_free(device->host_allocator, device);
}

static iree_string_view_t b200_device_id(iree_hal_device_t* base) { return b200_device_cast(base)->identifier; }
static iree_allocator_t b200_device_host_allocator(iree_hal_device_t* base) { return b200_device_cast(base)->host_allocator; }
static iree_hal_allocator_t* b200_device_allocator(iree_hal_device_t* base) { return b200_device_cast(base)->device_allocator; }

static void b200_device_replace_allocator(iree_hal_device_t* base, iree_hal_allocator_t* new_allocator) {
  b200_device_t* device = b200_device_cast(base);
  iree_hal_allocator_retain(new_allocator);
  iree_hal_allocator_release(device->device_allocator);
  device->device_allocator = new_allocator;
}

static void b200_device_replace_channel_provider(iree_hal_device_t* base, iree_hal_channel_provider_t* new_provider) {}

static iree_status_t b200_device_trim(iree_hal_device_t* base) {
  b200_device_t* device = b200_device_cast(base);
  iree_arena_block_pool_trim(&device->block_pool);
  return iree_hal_allocator_trim(device->device_allocator);
}

// "hal.executable.format" :: "torq-b200-ops" = 1 in place of the reference's "torq-fb"
// (torq_device.c:206-213); the other keys are answered by the library as well (concurrency = 1).
static iree_status_t b200_device_query_i64(iree_hal_device_t* base, iree_string_view_t category, iree_string_view_t key,
                                           int64_t* out_value) {
  b200_device_t* device = b200_device_cast(base);
  *out_value = 0;
  if (iree_string_view_equal(category, IREE_SV("hal.device.id"))) {
    *out_value = iree_string_view_match_pattern(device->identifier, key) ? 1 : 0;
    return iree_ok_status();
  }
  char category_z[64], key_z[64];
  if (category.size >= sizeof(category_z) || key.size >= sizeof(key_z)) {
    return iree_make_status(IREE_STATUS_NOT_FOUND, "unknown device configuration key value '%.*s :: %.*s'",
                            (int)category.size, category.data, (int)key.size, key.data);
  }
  memcpy(category_z, category.data, category.size);
  category_z[category.size] = 0;
  memcpy(key_z, key.data, key.size);
  key_z[key.size] = 0;
  B200_RETURN_IF_ERROR(device->handle, tb200_device_query_i64(device->handle, category_z, key_z, out_value));
  return iree_ok_status();
}

static iree_status_t b200_device_create_channel(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                                iree_hal_channel_params_t params, iree_hal_channel_t** out_channel) {
  return iree_make_status(IREE_STATUS_UNIMPLEMENTED, "collectives not implemented");
}

static iree_status_t b200_device_create_command_buffer(iree_hal_device_t* base, iree_hal_command_buffer_mode_t mode,
                                                       iree_hal_command_category_t command_categories,
                                                       iree_hal_queue_affinity_t queue_affinity,
                                                       iree_host_size_t binding_capacity,
                                                       iree_hal_command_buffer_t** out_command_buffer) {
  b200_device_t* device = b200_device_cast(base);
  if (iree_all_bits_set(mode, IREE_HAL_COMMAND_BUFFER_MODE_ONE_SHOT | IREE_HAL_COMMAND_BUFFER_MODE_ALLOW_INLINE_EXECUTION) &&
      binding_capacity == 0) {
    return iree_hal_torq_b200_command_buffer_create(device->device_allocator, device->handle, mode, command_categories,
                                                    queue_affinity, binding_capacity, device->host_allocator,
                                                    out_command_buffer);
  }
  return iree_hal_deferred_command_buffer_create(device->device_allocator, mode, command_categories, queue_affinity,
                                                 binding_capacity, &device->block_pool, device->host_allocator,
                                                 out_command_buffer);
}

static iree_status_t b200_device_create_event(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                              iree_hal_event_flags_t flags, iree_hal_event_t** out_event) {
  return iree_make_status(IREE_STATUS_UNIMPLEMENTED, "events are not needed on a single in-order stream");
}

static iree_status_t b200_device_create_executable_cache(iree_hal_device_t* base, iree_string_view_t identifier,
                                                         iree_loop_t loop, iree_hal_executable_cache_t** out_cache) {
  b200_device_t* device = b200_device_cast(base);
  return iree_hal_torq_b200_executable_cache_create(device->handle, identifier, device->host_allocator, out_cache);
}

static iree_status_t b200_device_import_file(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                             iree_hal_memory_access_t access, iree_io_file_handle_t* handle,
                                             iree_hal_external_file_flags_t flags, iree_hal_file_t** out_file) {
  return iree_hal_file_from_handle(iree_hal_device_allocator(base), queue_affinity, access, handle,
                                   iree_hal_device_host_allocator(base), out_file);
}

static iree_status_t b200_device_create_semaphore(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                                  uint64_t initial_value, iree_hal_semaphore_flags_t flags,
                                                  iree_hal_semaphore_t** out_semaphore) {
  return iree_hal_torq_b200_semaphore_create(initial_value, b200_device_cast(base)->host_allocator, out_semaphore);
}

static iree_hal_semaphore_compatibility_t b200_device_query_semaphore_compatibility(iree_hal_device_t* base,
                                                                                   iree_hal_semaphore_t* semaphore) {
  return iree_hal_torq_b200_semaphore_isa(semaphore) ? IREE_HAL_SEMAPHORE_COMPATIBILITY_ALL
                                                     : IREE_HAL_SEMAPHORE_COMPATIBILITY_HOST_ONLY;
}

//===-- queue operations -----------------------------------------------------
// Shape of every queue call: wait for the wait list, do the work, drain the stream, signal the signal list.

static iree_status_t b200_queue_finish(b200_device_t* device, iree_status_t status,
                                       const iree_hal_semaphore_list_t signal_semaphore_list) {
  if (iree_status_is_ok(status)) {
    // ABORTED here means a kernel gave up on one of its bounded waits (the reference's wait for the NPU has a
    // timeout too, runtime/torq_hw/src/TorqHw.cpp:172-186); the device stays usable
    status = iree_hal_torq_b200_status(tb200_wait(device->handle, UINT64_MAX), device->handle, "tb200_wait");
  }
  if (iree_status_is_ok(status)) return iree_hal_semaphore_list_signal(signal_semaphore_list);
  iree_hal_semaphore_list_fail(signal_semaphore_list, iree_status_clone(status));
  return status;
}

static iree_status_t b200_device_queue_alloca(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                              const iree_hal_semaphore_list_t wait_semaphore_list,
                                              const iree_hal_semaphore_list_t signal_semaphore_list,
                                              iree_hal_allocator_pool_t pool, iree_hal_buffer_params_t params,
                                              iree_device_size_t allocation_size, iree_hal_alloca_flags_t flags,
                                              iree_hal_buffer_t** IREE_RESTRICT out_buffer) {
  IREE_RETURN_IF_ERROR(iree_hal_semaphore_list_wait(wait_semaphore_list, iree_infinite_timeout(), IREE_HAL_WAIT_FLAG_DEFAULT));
  IREE_RETURN_IF_ERROR(iree_hal_allocator_allocate_buffer(iree_hal_device_allocator(base), params, allocation_size, out_buffer));
  return iree_hal_semaphore_list_signal(signal_semaphore_list);
}

static iree_status_t b200_device_queue_dealloca(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                                const iree_hal_semaphore_list_t wait_semaphore_list,
                                                const iree_hal_semaphore_list_t signal_semaphore_list,
                                                iree_hal_buffer_t* buffer, iree_hal_dealloca_flags_t flags) {
  // the buffer is freed when its last reference goes (tb200_buffer_free waits for the stream first)
  IREE_RETURN_IF_ERROR(iree_hal_semaphore_list_wait(wait_semaphore_list, iree_infinite_timeout(), IREE_HAL_WAIT_FLAG_DEFAULT));
  return iree_hal_semaphore_list_signal(signal_semaphore_list);
}

static iree_status_t b200_device_queue_read(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                            const iree_hal_semaphore_list_t wait_semaphore_list,
                                            const iree_hal_semaphore_list_t signal_semaphore_list,
                                            iree_hal_file_t* source_file, uint64_t source_offset,
                                            iree_hal_buffer_t* target_buffer, iree_device_size_t target_offset,
                                            iree_device_size_t length, iree_hal_read_flags_t flags) {
  iree_status_t loop_status = iree_ok_status();
  iree_hal_file_transfer_options_t options = {.loop = iree_loop_inline(&loop_status), .chunk_count = IREE_HAL_FILE_TRANSFER_CHUNK_COUNT_DEFAULT,
                                              .chunk_size = IREE_HAL_FILE_TRANSFER_CHUNK_SIZE_DEFAULT};
  IREE_RETURN_IF_ERROR(iree_hal_device_queue_read_streaming(base, queue_affinity, wait_semaphore_list, signal_semaphore_list,
                                                            source_file, source_offset, target_buffer, target_offset, length,
                                                            flags, options));
  return loop_status;
}

static iree_status_t b200_device_queue_write(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                             const iree_hal_semaphore_list_t wait_semaphore_list,
                                             const iree_hal_semaphore_list_t signal_semaphore_list,
                                             iree_hal_buffer_t* source_buffer, iree_device_size_t source_offset,
                                             iree_hal_file_t* target_file, uint64_t target_offset, iree_device_size_t length,
                                             iree_hal_write_flags_t flags) {
  iree_status_t loop_status = iree_ok_status();
  iree_hal_file_transfer_options_t options = {.loop = iree_loop_inline(&loop_status), .chunk_count = IREE_HAL_FILE_TRANSFER_CHUNK_COUNT_DEFAULT,
                                              .chunk_size = IREE_HAL_FILE_TRANSFER_CHUNK_SIZE_DEFAULT};
  IREE_RETURN_IF_ERROR(iree_hal_device_queue_write_streaming(base, queue_affinity, wait_semaphore_list, signal_semaphore_list,
                                                             source_buffer, source_offset, target_file, target_offset, length,
                                                             flags, options));
  return loop_status;
}

static iree_status_t b200_device_queue_host_call(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                                 const iree_hal_semaphore_list_t wait_semaphore_list,
                                                 const iree_hal_semaphore_list_t signal_semaphore_list,
                                                 iree_hal_host_call_t call, const uint64_t args[4],
                                                 iree_hal_host_call_flags_t flags) {
  b200_device_t* device = b200_device_cast(base);
  IREE_RETURN_IF_ERROR(iree_hal_semaphore_list_wait(wait_semaphore_list, iree_infinite_timeout(), IREE_HAL_WAIT_FLAG_DEFAULT));
  const bool non_blocking = iree_any_bit_set(flags, IREE_HAL_HOST_CALL_FLAG_NON_BLOCKING);
  if (non_blocking) IREE_RETURN_IF_ERROR(iree_hal_semaphore_list_signal(signal_semaphore_list));
  iree_hal_host_call_context_t context = {
      .device = base,
      .queue_affinity = queue_affinity,
      .signal_semaphore_list = non_blocking ? iree_hal_semaphore_list_empty() : signal_semaphore_list,
  };
  iree_status_t status = call.fn(call.user_data, args, &context);
  if (non_blocking) {
    iree_status_ignore(status);
    return iree_ok_status();
  }
  if (iree_status_is_deferred(status)) return iree_ok_status();  // the callee signals
  return b200_queue_finish(device, status, signal_semaphore_list);
}

// Deferred (reusable / indirect) command buffers are replayed into an inline one of this driver.
static iree_status_t b200_apply_deferred(b200_device_t* device, iree_hal_command_buffer_t* command_buffer,
                                         iree_hal_buffer_binding_table_t binding_table) {
  if (!command_buffer || !iree_hal_deferred_command_buffer_isa(command_buffer)) return iree_ok_status();  // ran inline
  iree_hal_command_buffer_t* inline_buffer = NULL;
  IREE_RETURN_IF_ERROR(iree_hal_torq_b200_command_buffer_create(
      device->device_allocator, device->handle,
      iree_hal_command_buffer_mode(command_buffer) | IREE_HAL_COMMAND_BUFFER_MODE_ONE_SHOT |
          IREE_HAL_COMMAND_BUFFER_MODE_ALLOW_INLINE_EXECUTION |
          (iree_hal_buffer_binding_table_is_empty(binding_table) ? IREE_HAL_COMMAND_BUFFER_MODE_UNVALIDATED : 0),
      iree_hal_command_buffer_allowed_categories(command_buffer), IREE_HAL_QUEUE_AFFINITY_ANY, /*binding_capacity=*/0,
      device->host_allocator, &inline_buffer));
  iree_status_t status = iree_hal_deferred_command_buffer_apply(command_buffer, inline_buffer, binding_table);
  iree_hal_command_buffer_release(inline_buffer);
  return status;
}

static iree_status_t b200_device_queue_execute(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity,
                                               const iree_hal_semaphore_list_t wait_semaphore_list,
                                               const iree_hal_semaphore_list_t signal_semaphore_list,
                                               iree_hal_command_buffer_t* command_buffer,
                                               iree_hal_buffer_binding_table_t binding_table, iree_hal_execute_flags_t flags) {
  b200_device_t* device = b200_device_cast(base);
  iree_status_t status = iree_hal_semaphore_list_wait(wait_semaphore_list, iree_infinite_timeout(), IREE_HAL_WAIT_FLAG_DEFAULT);
  if (iree_status_is_ok(status)) status = b200_apply_deferred(device, command_buffer, binding_table);
  return b200_queue_finish(device, status, signal_semaphore_list);
}

static iree_status_t b200_device_queue_flush(iree_hal_device_t* base, iree_hal_queue_affinity_t queue_affinity) {
  return iree_ok_status();  // launches are submitted as they are recorded
}

static iree_status_t b200_device_wait_semaphores(iree_hal_device_t* base, iree_hal_wait_mode_t wait_mode,
                                                 const iree_hal_semaphore_list_t semaphore_list, iree_timeout_t timeout,
                                                 iree_hal_wait_flags_t flags) {
  return iree_hal_torq_b200_semaphore_multi_wait(wait_mode, semaphore_list, timeout);
}

// --torq_profile_host=<csv> of the reference (runtime/torq_hw/src/TorqEventLog.cpp:23) maps to
// tb200_device_set_profile_csv: same columns and event names. The HAL profiling slots switch it on a
// file named by the options.
static iree_status_t b200_device_profiling_begin(iree_hal_device_t* base, const iree_hal_device_profiling_options_t* options) {
  b200_device_t* device = b200_device_cast(base);
  if (options->file_path && options->file_path[0]) {
    B200_RETURN_IF_ERROR(device->handle, tb200_device_set_profile_csv(device->handle, options->file_path));
  }
  return iree_ok_status();
}
static iree_status_t b200_device_profiling_flush(iree_hal_device_t* base) { return iree_ok_status(); }
static iree_status_t b200_device_profiling_end(iree_hal_device_t* base) {
  b200_device_t* device = b200_device_cast(base);
  B200_RETURN_IF_ERROR(device->handle, tb200_device_set_profile_csv(device->handle, NULL));
  return iree_ok_status();
}

static const iree_hal_device_vtable_t b200_device_vtable = {
    .destroy = b200_device_destroy,
    .id = b200_device_id,
    .host_allocator = b200_device_host_allocator,
    .device_allocator = b200_device_allocator,
    .replace_device_allocator = b200_device_replace_allocator,
    .replace_channel_provider = b200_device_replace_channel_provider,
    .trim = b200_device_trim,
    .query_i64 = b200_device_query_i64,
    .create_channel = b200_device_create_channel,
    .create_command_buffer = b200_device_create_command_buffer,
    .create_event = b200_device_create_event,
    .create_executable_cache = b200_device_create_executable_cache,
    .import_file = b200_device_import_file,
    .create_semaphore = b200_device_create_semaphore,
    .query_semaphore_compatibility = b200_device_query_semaphore_compatibility,
    .queue_alloca = b200_device_queue_alloca,
    .queue_dealloca = b200_device_queue_dealloca,
    .queue_fill = iree_hal_device_queue_emulated_fill,
    .queue_update = iree_hal_device_queue_emulated_update,
    .queue_copy = iree_hal_device_queue_emulated_copy,
    .queue_read = b200_device_queue_read,
    .queue_write = b200_device_queue_write,
    .queue_host_call = b200_device_queue_host_call,
    .queue_dispatch = iree_hal_device_queue_emulated_dispatch,
    .queue_execute = b200_device_queue_execute,
    .queue_flush = b200_device_queue_flush,
    .wait_semaphores = b200_device_wait_semaphores,
    .profiling_begin = b200_device_profiling_begin,
    .profiling_flush = b200_device_profiling_flush,
    .profiling_end = b200_device_profiling_end,
};
