// Allocator and buffers of the torq_b200 HAL driver. Slots as in runtime/driver/torq_allocator.c:398-418 of
// the reference, but with the two heaps of a discrete GPU: DEVICE_LOCAL (HBM, tb200_buffer_alloc
// TB200_MEMORY_DEVICE_LOCAL; not host-visible) and HOST_VISIBLE | HOST_COHERENT pinned staging
// (TB200_MEMORY_HOST_PINNED; mappable, transfer only). The reference has one heap that is both
// (torq_allocator.c:182-207) because its NPU shares the host's memory.
// Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"

typedef struct b200_allocator_t {
  iree_hal_resource_t resource;
  iree_allocator_t host_allocator;
  tb200_device_t* device;
  iree_hal_allocator_statistics_t statistics;
} b200_allocator_t;

typedef struct b200_buffer_t {
  iree_hal_buffer_t base;
  iree_allocator_t host_allocator;
  tb200_buffer_t* handle;
  bool host_visible;
  iree_hal_buffer_release_callback_t release_callback;  // imported buffers
} b200_buffer_t;

static const iree_hal_allocator_vtable_t b200_allocator_vtable;
static const iree_hal_buffer_vtable_t b200_buffer_vtable;

tb200_buffer_t* iree_hal_torq_b200_buffer_handle(iree_hal_buffer_t* buffer) {
  iree_hal_buffer_t* allocated = iree_hal_buffer_allocated_buffer(buffer);
  if (!iree_hal_resource_is(&allocated->resource, &b200_buffer_vtable)) return NULL;
  return ((b200_buffer_t*)allocated)->handle;
}

//===-- buffer ---------------------------------------------------------------

static void b200_buffer_destroy(iree_hal_buffer_t* base_buffer) {
  b200_buffer_t* buffer = (b200_buffer_t*)base_buffer;
  if (buffer->release_callback.fn) buffer->release_callback.fn(buffer->release_callback.user_data, base_buffer);
  if (buffer->handle) tb200_buffer_free(buffer->handle);
  iree_allocator_free(buffer->host_allocator, buffer);
}

// Only the pinned staging heap maps; HBM is reached through transfer commands.
static iree_status_t b200_buffer_map_range(iree_hal_buffer_t* base_buffer, iree_hal_mapping_mode_t mapping_mode,
                                           iree_hal_memory_access_t memory_access, iree_device_size_t local_byte_offset,
                                           iree_device_size_t local_byte_length, iree_hal_buffer_mapping_t* mapping) {
  b200_buffer_t* buffer = (b200_buffer_t*)base_buffer;
  if (!buffer->host_visible) {
    return iree_make_status(IREE_STATUS_FAILED_PRECONDITION,
                            "device-local buffers of torq_b200 live in HBM and cannot be mapped; use a transfer command");
  }
  mapping->contents = iree_make_byte_span((uint8_t*)tb200_buffer_pointer(buffer->handle) + local_byte_offset,
                                          local_byte_length);
  return iree_ok_status();
}

static iree_status_t b200_buffer_unmap_range(iree_hal_buffer_t* base_buffer, iree_device_size_t local_byte_offset,
                                             iree_device_size_t local_byte_length, iree_hal_buffer_mapping_t* mapping) {
  return iree_ok_status();
}

static iree_status_t b200_buffer_invalidate_range(iree_hal_buffer_t* base_buffer, iree_device_size_t local_byte_offset,
                                                  iree_device_size_t local_byte_length) {
  return iree_ok_status();  // pinned memory is coherent
}

static iree_status_t b200_buffer_flush_range(iree_hal_buffer_t* base_buffer, iree_device_size_t local_byte_offset,
                                             iree_device_size_t local_byte_length) {
  return iree_ok_status();
}

static iree_status_t b200_buffer_wrap(b200_allocator_t* allocator, const iree_hal_buffer_params_t* params,
                                      iree_device_size_t size, tb200_buffer_t* handle, bool host_visible,
                                      iree_hal_buffer_release_callback_t release_callback, iree_hal_buffer_t** out_buffer) {
  b200_buffer_t* buffer = NULL;
  iree_status_t status = iree_allocator_malloc(allocator->host_allocator, sizeof(*buffer), (void**)&buffer);
  if (!iree_status_is_ok(status)) {
    tb200_buffer_free(handle);
    return status;
  }
  buffer->host_allocator = allocator->host_allocator;
  buffer->handle = handle;
  buffer->host_visible = host_visible;
  buffer->release_callback = release_callback;
  const iree_hal_buffer_placement_t placement = {
      .device = NULL,
      .queue_affinity = params->queue_affinity ? params->queue_affinity : IREE_HAL_QUEUE_AFFINITY_ANY,
      .flags = IREE_HAL_BUFFER_PLACEMENT_FLAG_NONE,
  };
  iree_hal_buffer_initialize(placement, &buffer->base, size, 0, size, params->type, params->access, params->usage,
                             &b200_buffer_vtable, &buffer->base);
  *out_buffer = &buffer->base;
  return iree_ok_status();
}

//===-- allocator ------------------------------------------------------------

iree_status_t iree_hal_torq_b200_allocator_create(tb200_device_t* device, iree_allocator_t host_allocator,
                                                  iree_hal_allocator_t** out_allocator) {
  *out_allocator = NULL;
  b200_allocator_t* allocator = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, sizeof(*allocator), (void**)&allocator));
  iree_hal_resource_initialize(&b200_allocator_vtable, &allocator->resource);
  allocator->host_allocator = host_allocator;
  allocator->device = device;
  memset(&allocator->statistics, 0, sizeof(allocator->statistics));
  *out_allocator = (iree_hal_allocator_t*)allocator;
  return iree_ok_status();
}

static void b200_allocator_destroy(iree_hal_allocator_t* base_allocator) {
  b200_allocator_t* allocator = (b200_allocator_t*)base_allocator;
  iree_allocator_free(allocator->host_allocator, allocator);
}

static iree_allocator_t b200_allocator_host_allocator(const iree_hal_allocator_t* base_allocator) {
  return ((const b200_allocator_t*)base_allocator)->host_allocator;
}

static iree_status_t b200_allocator_trim(iree_hal_allocator_t* base_allocator) { return iree_ok_status(); }

static void b200_allocator_query_statistics(iree_hal_allocator_t* base_allocator,
                                            iree_hal_allocator_statistics_t* out_statistics) {
  *out_statistics = ((b200_allocator_t*)base_allocator)->statistics;
}

static iree_status_t b200_allocator_query_memory_heaps(iree_hal_allocator_t* base_allocator, iree_host_size_t capacity,
                                                       iree_hal_allocator_memory_heap_t* heaps,
                                                       iree_host_size_t* out_count) {
  const iree_host_size_t count = 2;
  if (out_count) *out_count = count;
  if (capacity < count) return iree_status_from_code(IREE_STATUS_OUT_OF_RANGE);
  heaps[0] = (iree_hal_allocator_memory_heap_t){
      .type = IREE_HAL_MEMORY_TYPE_DEVICE_LOCAL,
      .allowed_usage = IREE_HAL_BUFFER_USAGE_TRANSFER | IREE_HAL_BUFFER_USAGE_DISPATCH,
      .max_allocation_size = ~(iree_device_size_t)0,
      .min_alignment = 256,  // cudaMalloc's; the kernels want 16
  };
  heaps[1] = (iree_hal_allocator_memory_heap_t){
      .type = IREE_HAL_MEMORY_TYPE_HOST_LOCAL | IREE_HAL_MEMORY_TYPE_HOST_COHERENT | IREE_HAL_MEMORY_TYPE_DEVICE_VISIBLE,
      .allowed_usage = IREE_HAL_BUFFER_USAGE_TRANSFER | IREE_HAL_BUFFER_USAGE_MAPPING,
      .max_allocation_size = ~(iree_device_size_t)0,
      .min_alignment = 64,
  };
  return iree_ok_status();
}

static bool b200_wants_host_heap(const iree_hal_buffer_params_t* params) {
  return iree_any_bit_set(params->type, IREE_HAL_MEMORY_TYPE_HOST_VISIBLE) ||
         iree_any_bit_set(params->usage, IREE_HAL_BUFFER_USAGE_MAPPING);
}

static iree_hal_buffer_compatibility_t b200_allocator_query_buffer_compatibility(iree_hal_allocator_t* base_allocator,
                                                                                 iree_hal_buffer_params_t* params,
                                                                                 iree_device_size_t* allocation_size) {
  iree_hal_buffer_compatibility_t compatibility =
      IREE_HAL_BUFFER_COMPATIBILITY_ALLOCATABLE | IREE_HAL_BUFFER_COMPATIBILITY_IMPORTABLE;
  if (iree_any_bit_set(params->usage, IREE_HAL_BUFFER_USAGE_TRANSFER))
    compatibility |= IREE_HAL_BUFFER_COMPATIBILITY_QUEUE_TRANSFER;
  if (b200_wants_host_heap(params)) {
    // staging memory: a dispatch cannot bind it (tb200_dispatch answers FAILED_PRECONDITION)
    params->type |= IREE_HAL_MEMORY_TYPE_HOST_LOCAL | IREE_HAL_MEMORY_TYPE_HOST_COHERENT | IREE_HAL_MEMORY_TYPE_DEVICE_VISIBLE;
    params->type &= ~IREE_HAL_MEMORY_TYPE_DEVICE_LOCAL;
    params->usage &= ~IREE_HAL_BUFFER_USAGE_DISPATCH;
  } else {
    params->type |= IREE_HAL_MEMORY_TYPE_DEVICE_LOCAL;
    if (iree_any_bit_set(params->usage, IREE_HAL_BUFFER_USAGE_DISPATCH_STORAGE))
      compatibility |= IREE_HAL_BUFFER_COMPATIBILITY_QUEUE_DISPATCH;
  }
  params->type &= ~IREE_HAL_MEMORY_TYPE_OPTIMAL;
  if (*allocation_size == 0) *allocation_size = 16;
  *allocation_size = iree_host_align(*allocation_size, 16);
  return compatibility;
}

static iree_status_t b200_allocator_allocate_buffer(iree_hal_allocator_t* base_allocator,
                                                    const iree_hal_buffer_params_t* params,
                                                    iree_device_size_t allocation_size, iree_hal_buffer_t** out_buffer) {
  b200_allocator_t* allocator = (b200_allocator_t*)base_allocator;
  iree_hal_buffer_params_t compat_params = *params;
  if (!iree_all_bits_set(b200_allocator_query_buffer_compatibility(base_allocator, &compat_params, &allocation_size),
                         IREE_HAL_BUFFER_COMPATIBILITY_ALLOCATABLE)) {
    return iree_make_status(IREE_STATUS_INVALID_ARGUMENT, "allocator cannot allocate a buffer with these parameters");
  }
  const bool host = b200_wants_host_heap(&compat_params);
  tb200_buffer_t* handle = NULL;
  B200_RETURN_IF_ERROR(allocator->device,
                       tb200_buffer_alloc(allocator->device, allocation_size,
                                          host ? TB200_MEMORY_HOST_PINNED : TB200_MEMORY_DEVICE_LOCAL, &handle));
  iree_hal_buffer_release_callback_t no_callback = {0};
  return b200_buffer_wrap(allocator, &compat_params, allocation_size, handle, host, no_callback, out_buffer);
}

static void b200_allocator_deallocate_buffer(iree_hal_allocator_t* base_allocator, iree_hal_buffer_t* base_buffer) {
  iree_hal_buffer_destroy(base_buffer);
}

// A CUDA device pointer of the same GPU handed in by the host program becomes a bindable buffer
// without a copy (tb200_buffer_import); the caller keeps ownership.
static iree_status_t b200_allocator_import_buffer(iree_hal_allocator_t* base_allocator,
                                                  const iree_hal_buffer_params_t* params,
                                                  iree_hal_external_buffer_t* external_buffer,
                                                  iree_hal_buffer_release_callback_t release_callback,
                                                  iree_hal_buffer_t** out_buffer) {
  b200_allocator_t* allocator = (b200_allocator_t*)base_allocator;
  if (external_buffer->type != IREE_HAL_EXTERNAL_BUFFER_TYPE_DEVICE_ALLOCATION) {
    return iree_make_status(IREE_STATUS_UNAVAILABLE, "torq_b200 imports device allocations (CUDA device pointers) only");
  }
  tb200_buffer_t* handle = NULL;
  B200_RETURN_IF_ERROR(allocator->device,
                       tb200_buffer_import(allocator->device, (void*)(uintptr_t)external_buffer->handle.device_allocation.ptr,
                                           external_buffer->size, &handle));
  iree_hal_buffer_params_t compat_params = *params;
  compat_params.type |= IREE_HAL_MEMORY_TYPE_DEVICE_LOCAL;
  return b200_buffer_wrap(allocator, &compat_params, external_buffer->size, handle, false, release_callback, out_buffer);
}

static iree_status_t b200_allocator_export_buffer(iree_hal_allocator_t* base_allocator, iree_hal_buffer_t* buffer,
                                                  iree_hal_external_buffer_type_t requested_type,
                                                  iree_hal_external_buffer_flags_t requested_flags,
                                                  iree_hal_external_buffer_t* out_external_buffer) {
  tb200_buffer_t* handle = iree_hal_torq_b200_buffer_handle(buffer);
  if (!handle || requested_type != IREE_HAL_EXTERNAL_BUFFER_TYPE_DEVICE_ALLOCATION) {
    return iree_make_status(IREE_STATUS_UNAVAILABLE, "torq_b200 exports its own buffers as device allocations only");
  }
  out_external_buffer->type = requested_type;
  out_external_buffer->flags = requested_flags;
  out_external_buffer->size = (iree_device_size_t)tb200_buffer_size(handle);
  out_external_buffer->handle.device_allocation.ptr = (uint64_t)(uintptr_t)tb200_buffer_pointer(handle);
  return iree_ok_status();
}

static const iree_hal_allocator_vtable_t b200_allocator_vtable = {
    .destroy = b200_allocator_destroy,
    .host_allocator = b200_allocator_host_allocator,
    .trim = b200_allocator_trim,
    .query_statistics = b200_allocator_query_statistics,
    .query_memory_heaps = b200_allocator_query_memory_heaps,
    .query_buffer_compatibility = b200_allocator_query_buffer_compatibility,
    .allocate_buffer = b200_allocator_allocate_buffer,
    .deallocate_buffer = b200_allocator_deallocate_buffer,
    .import_buffer = b200_allocator_import_buffer,
    .export_buffer = b200_allocator_export_buffer,
};

static const iree_hal_buffer_vtable_t b200_buffer_vtable = {
    .recycle = iree_hal_buffer_recycle,
    .destroy = b200_buffer_destroy,
    .map_range = b200_buffer_map_range,
    .unmap_range = b200_buffer_unmap_range,
    .invalidate_range = b200_buffer_invalidate_range,
    .flush_range = b200_buffer_flush_range,
};
