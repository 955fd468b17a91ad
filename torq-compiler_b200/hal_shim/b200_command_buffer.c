// Command buffer of the torq_b200 HAL driver. Like the reference's (runtime/driver/torq_command_buffer.c) it
// executes inline as it is recorded; unlike the reference's, commands are stream operations on the device
// (the C ABI's calls only enqueue), so "inline" costs the host one enqueue per command. The 15 slots are
// those of torq_command_buffer.c:514-531. Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"

#define B200_MAX_BINDINGS 64

typedef struct b200_command_buffer_t {
  iree_hal_command_buffer_t base;
  iree_allocator_t host_allocator;
  tb200_device_t* device;
} b200_command_buffer_t;

static const iree_hal_command_buffer_vtable_t b200_command_buffer_vtable;

bool iree_hal_torq_b200_command_buffer_isa(iree_hal_command_buffer_t* command_buffer) {
  return iree_hal_resource_is(&command_buffer->resource, &b200_command_buffer_vtable);
}

iree_status_t iree_hal_torq_b200_command_buffer_create(iree_hal_allocator_t* device_allocator, tb200_device_t* device,
                                                       iree_hal_command_buffer_mode_t mode,
                                                       iree_hal_command_category_t command_categories,
                                                       iree_hal_queue_affinity_t queue_affinity,
                                                       iree_host_size_t binding_capacity, iree_allocator_t host_allocator,
                                                       iree_hal_command_buffer_t** out_command_buffer) {
  *out_command_buffer = NULL;
  // Inline execution only: one-shot, no indirect binding tables. Reusable command buffers are recorded
  // by iree_hal_deferred_command_buffer_t and replayed into one of these (b200_device.c).
  if (!iree_all_bits_set(mode, IREE_HAL_COMMAND_BUFFER_MODE_ONE_SHOT | IREE_HAL_COMMAND_BUFFER_MODE_ALLOW_INLINE_EXECUTION)) {
    return iree_make_status(IREE_STATUS_INVALID_ARGUMENT, "inline command buffers must be one-shot and allow inline execution");
  }
  if (binding_capacity > 0) {
    return iree_make_status(IREE_STATUS_INVALID_ARGUMENT, "indirect bindings need a deferred command buffer");
  }
  b200_command_buffer_t* command_buffer = NULL;
  const iree_host_size_t total =
      sizeof(*command_buffer) + iree_hal_command_buffer_validation_state_size(mode, binding_capacity);
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, total, (void**)&command_buffer));
  iree_hal_command_buffer_initialize(device_allocator, mode, command_categories, queue_affinity, binding_capacity,
                                     (uint8_t*)command_buffer + sizeof(*command_buffer), &b200_command_buffer_vtable,
                                     &command_buffer->base);
  command_buffer->host_allocator = host_allocator;
  command_buffer->device = device;
  *out_command_buffer = &command_buffer->base;
  return iree_ok_status();
}

static void b200_command_buffer_destroy(iree_hal_command_buffer_t* base) {
  b200_command_buffer_t* command_buffer = (b200_command_buffer_t*)base;
  iree_allocator_free(command_buffer->host_allocator, command_buffer);
}

static iree_status_t b200_command_buffer_begin(iree_hal_command_buffer_t* base) { return iree_ok_status(); }
static iree_status_t b200_command_buffer_end(iree_hal_command_buffer_t* base) { return iree_ok_status(); }

static iree_status_t b200_command_buffer_begin_debug_group(iree_hal_command_buffer_t* base, iree_string_view_t label,
                                                           iree_hal_label_color_t label_color,
                                                           const iree_hal_label_location_t* location) {
  return iree_ok_status();
}
static iree_status_t b200_command_buffer_end_debug_group(iree_hal_command_buffer_t* base) { return iree_ok_status(); }

// Everything is ordered by the one device stream: barriers and events have nothing left to do.
static iree_status_t b200_command_buffer_execution_barrier(iree_hal_command_buffer_t* base,
                                                           iree_hal_execution_stage_t source_stage_mask,
                                                           iree_hal_execution_stage_t target_stage_mask,
                                                           iree_hal_execution_barrier_flags_t flags,
                                                           iree_host_size_t memory_barrier_count,
                                                           const iree_hal_memory_barrier_t* memory_barriers,
                                                           iree_host_size_t buffer_barrier_count,
                                                           const iree_hal_buffer_barrier_t* buffer_barriers) {
  return iree_ok_status();
}
static iree_status_t b200_command_buffer_signal_event(iree_hal_command_buffer_t* base, iree_hal_event_t* event,
                                                      iree_hal_execution_stage_t source_stage_mask) {
  return iree_ok_status();
}
static iree_status_t b200_command_buffer_reset_event(iree_hal_command_buffer_t* base, iree_hal_event_t* event,
                                                     iree_hal_execution_stage_t source_stage_mask) {
  return iree_ok_status();
}
static iree_status_t b200_command_buffer_wait_events(iree_hal_command_buffer_t* base, iree_host_size_t event_count,
                                                     const iree_hal_event_t** events,
                                                     iree_hal_execution_stage_t source_stage_mask,
                                                     iree_hal_execution_stage_t target_stage_mask,
                                                     iree_host_size_t memory_barrier_count,
                                                     const iree_hal_memory_barrier_t* memory_barriers,
                                                     iree_host_size_t buffer_barrier_count,
                                                     const iree_hal_buffer_barrier_t* buffer_barriers) {
  return iree_ok_status();
}
static iree_status_t b200_command_buffer_advise_buffer(iree_hal_command_buffer_t* base, iree_hal_buffer_ref_t buffer_ref,
                                                       iree_hal_memory_advise_flags_t flags, uint64_t arg0, uint64_t arg1) {
  return iree_ok_status();
}

// A (buffer, offset) reference resolved to a C-ABI buffer and a byte offset inside it.
static iree_status_t b200_resolve(iree_hal_buffer_ref_t ref, tb200_buffer_t** out_handle, uint64_t* out_offset) {
  if (!ref.buffer) {
    return iree_make_status(IREE_STATUS_FAILED_PRECONDITION, "buffer reference is NULL");
  }
  *out_handle = iree_hal_torq_b200_buffer_handle(ref.buffer);
  if (!*out_handle) {
    return iree_make_status(IREE_STATUS_FAILED_PRECONDITION, "buffer was not allocated by the torq_b200 allocator");
  }
  *out_offset = (uint64_t)(iree_hal_buffer_byte_offset(ref.buffer) + ref.offset);
  return iree_ok_status();
}

// Transfers: the reference maps and memcpy()s (torq_command_buffer.c:332-373); here they are stream copies.
static iree_status_t b200_command_buffer_update_buffer(iree_hal_command_buffer_t* base, const void* source_buffer,
                                                       iree_host_size_t source_offset, iree_hal_buffer_ref_t target_ref,
                                                       iree_hal_update_flags_t flags) {
  b200_command_buffer_t* command_buffer = (b200_command_buffer_t*)base;
  tb200_buffer_t* target = NULL;
  uint64_t offset = 0;
  IREE_RETURN_IF_ERROR(b200_resolve(target_ref, &target, &offset));
  B200_RETURN_IF_ERROR(command_buffer->device,
                       tb200_buffer_upload(target, offset, (const uint8_t*)source_buffer + source_offset, target_ref.length));
  // the source is host memory the caller may reuse at once: the copy must have left it
  B200_RETURN_IF_ERROR(command_buffer->device, tb200_wait(command_buffer->device, UINT64_MAX));
  return iree_ok_status();
}

static iree_status_t b200_command_buffer_fill_buffer(iree_hal_command_buffer_t* base, iree_hal_buffer_ref_t target_ref,
                                                     const void* pattern, iree_host_size_t pattern_length,
                                                     iree_hal_fill_flags_t flags) {
  b200_command_buffer_t* command_buffer = (b200_command_buffer_t*)base;
  tb200_buffer_t* target = NULL;
  uint64_t offset = 0;
  IREE_RETURN_IF_ERROR(b200_resolve(target_ref, &target, &offset));
  // built on the upload path: a host-side pattern block repeated over the range
  uint8_t block[4096];
  for (iree_host_size_t i = 0; i < sizeof(block); i += pattern_length) memcpy(block + i, pattern, pattern_length);
  for (iree_device_size_t done = 0; done < target_ref.length; done += sizeof(block)) {
    const iree_device_size_t n = iree_min((iree_device_size_t)sizeof(block), target_ref.length - done);
    B200_RETURN_IF_ERROR(command_buffer->device, tb200_buffer_upload(target, offset + done, block, n));
  }
  B200_RETURN_IF_ERROR(command_buffer->device, tb200_wait(command_buffer->device, UINT64_MAX));
  return iree_ok_status();
}

static iree_status_t b200_command_buffer_copy_buffer(iree_hal_command_buffer_t* base, iree_hal_buffer_ref_t source_ref,
                                                     iree_hal_buffer_ref_t target_ref, iree_hal_copy_flags_t flags) {
  b200_command_buffer_t* command_buffer = (b200_command_buffer_t*)base;
  tb200_buffer_t *source = NULL, *target = NULL;
  uint64_t source_offset = 0, target_offset = 0;
  IREE_RETURN_IF_ERROR(b200_resolve(source_ref, &source, &source_offset));
  IREE_RETURN_IF_ERROR(b200_resolve(target_ref, &target, &target_offset));
  // tb200_buffer_upload copies from any address the device can read (host or device: cudaMemcpyDefault)
  B200_RETURN_IF_ERROR(command_buffer->device,
                       tb200_buffer_upload(target, target_offset, (const uint8_t*)tb200_buffer_pointer(source) + source_offset,
                                           source_ref.length));
  return iree_ok_status();
}

static iree_status_t b200_command_buffer_collective(iree_hal_command_buffer_t* base, iree_hal_channel_t* channel,
                                                    iree_hal_collective_op_t op, uint32_t param, iree_hal_buffer_ref_t send_ref,
                                                    iree_hal_buffer_ref_t recv_ref, iree_device_size_t element_count) {
  return iree_make_status(IREE_STATUS_UNIMPLEMENTED,
                          "collectives are not a HAL command of this driver: tensor-parallel executables exchange inside "
                          "their kernels (tb200_executable_connect_peers)");
}

// The hot path: one torq-b200-ops executable = one dispatch (the compiler emits a single dispatch per
// model, compiler/torq/Pipelines/InputConversionPassPipelines.cpp:73-78). Bindings are (buffer, offset,
// length) exactly as in the reference (torq_command_buffer.c:390-508); they are validated by the
// library with the reference's status codes and never mapped.
static iree_status_t b200_command_buffer_dispatch(iree_hal_command_buffer_t* base, iree_hal_executable_t* executable,
                                                  iree_hal_executable_export_ordinal_t export_ordinal,
                                                  const iree_hal_dispatch_config_t config, iree_const_byte_span_t constants,
                                                  iree_hal_buffer_ref_list_t bindings, iree_hal_dispatch_flags_t flags) {
  b200_command_buffer_t* command_buffer = (b200_command_buffer_t*)base;
  if (iree_hal_dispatch_uses_custom_arguments(flags)) {
    return iree_make_status(IREE_STATUS_UNIMPLEMENTED, "direct/indirect arguments are not supported on the torq_b200 command buffer");
  }
  if (IREE_UNLIKELY((constants.data_length % sizeof(uint32_t)) != 0)) {
    return iree_make_status(IREE_STATUS_FAILED_PRECONDITION, "constants must be 4-byte aligned");
  }
  if (export_ordinal != 0) {
    return iree_make_status(IREE_STATUS_OUT_OF_RANGE, "a torq-b200-ops executable has one entry point");
  }
  if (bindings.count > B200_MAX_BINDINGS) {
    return iree_make_status(IREE_STATUS_OUT_OF_RANGE, "more than %d bindings", B200_MAX_BINDINGS);
  }
  tb200_binding_t list[B200_MAX_BINDINGS];
  for (iree_host_size_t i = 0; i < bindings.count; ++i) {
    iree_hal_buffer_ref_t ref = bindings.values[i];
    list[i].buffer = ref.buffer ? iree_hal_torq_b200_buffer_handle(ref.buffer) : NULL;  // NULL -> FAILED_PRECONDITION below
    list[i].offset = ref.buffer ? (uint64_t)(iree_hal_buffer_byte_offset(ref.buffer) + ref.offset) : 0;
    list[i].length = ref.length == IREE_HAL_WHOLE_BUFFER ? 0 : (uint64_t)ref.length;
  }
  B200_RETURN_IF_ERROR(command_buffer->device,
                       tb200_dispatch(iree_hal_torq_b200_executable_handle(executable), list, bindings.count));
  return iree_ok_status();
}

static const iree_hal_command_buffer_vtable_t b200_command_buffer_vtable = {
    .destroy = b200_command_buffer_destroy,
    .begin = b200_command_buffer_begin,
    .end = b200_command_buffer_end,
    .begin_debug_group = b200_command_buffer_begin_debug_group,
    .end_debug_group = b200_command_buffer_end_debug_group,
    .execution_barrier = b200_command_buffer_execution_barrier,
    .signal_event = b200_command_buffer_signal_event,
    .reset_event = b200_command_buffer_reset_event,
    .wait_events = b200_command_buffer_wait_events,
    .advise_buffer = b200_command_buffer_advise_buffer,
    .fill_buffer = b200_command_buffer_fill_buffer,
    .update_buffer = b200_command_buffer_update_buffer,
    .copy_buffer = b200_command_buffer_copy_buffer,
    .collective = b200_command_buffer_collective,
    .dispatch = b200_command_buffer_dispatch,
};
