// Executable cache and executable of the torq_b200 HAL driver: the cache answers for the
// "torq-b200-ops" format and hands the blob to tb200_executable_create, which validates it, uploads its
// constants once and plans the launches. Slots as in runtime/driver/nop_executable_cache.cc:126-133 and
// runtime/driver/native_executable.cc:192-196 of the reference.
// Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"

//===-- executable -----------------------------------------------------------

typedef struct b200_executable_t {
  iree_hal_resource_t resource;
  iree_allocator_t host_allocator;
  tb200_executable_t* handle;
} b200_executable_t;

static const iree_hal_executable_vtable_t b200_executable_vtable;

tb200_executable_t* iree_hal_torq_b200_executable_handle(iree_hal_executable_t* executable) {
  IREE_HAL_ASSERT_TYPE(executable, &b200_executable_vtable);
  return ((b200_executable_t*)executable)->handle;
}

static iree_status_t b200_executable_create(tb200_device_t* device, iree_allocator_t host_allocator,
                                            const iree_hal_executable_params_t* params,
                                            iree_hal_executable_t** out_executable) {
  *out_executable = NULL;
  b200_executable_t* executable = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, sizeof(*executable), (void**)&executable));
  iree_hal_resource_initialize(&b200_executable_vtable, &executable->resource);
  executable->host_allocator = host_allocator;
  executable->handle = NULL;
  // The library copies what it keeps (as the reference copies the flatbuffer, native_executable.cc:62-63):
  // the caller's bytes need not outlive this call. Format and version mismatches come back as NOT_FOUND /
  // UNAVAILABLE, the reference's codes (nop_executable_cache.cc:97-105, TorqExecutable.cc:663-667).
  const int status = tb200_executable_create(device, params->executable_data.data, params->executable_data.data_length,
                                             &executable->handle);
  if (status != TB200_OK) {
    iree_allocator_free(host_allocator, executable);
    return iree_hal_torq_b200_status(status, device, "tb200_executable_create");
  }
  *out_executable = (iree_hal_executable_t*)executable;
  return iree_ok_status();
}

static void b200_executable_destroy(iree_hal_executable_t* base_executable) {
  b200_executable_t* executable = (b200_executable_t*)base_executable;
  if (executable->handle) tb200_executable_destroy(executable->handle);
  iree_allocator_free(executable->host_allocator, executable);
}

static const iree_hal_executable_vtable_t b200_executable_vtable = {
    .destroy = b200_executable_destroy,
};

//===-- executable cache -----------------------------------------------------

typedef struct b200_executable_cache_t {
  iree_hal_resource_t resource;
  iree_allocator_t host_allocator;
  tb200_device_t* device;
} b200_executable_cache_t;

static const iree_hal_executable_cache_vtable_t b200_executable_cache_vtable;

iree_status_t iree_hal_torq_b200_executable_cache_create(tb200_device_t* device, iree_string_view_t identifier,
                                                         iree_allocator_t host_allocator,
                                                         iree_hal_executable_cache_t** out_executable_cache) {
  *out_executable_cache = NULL;
  b200_executable_cache_t* cache = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, sizeof(*cache), (void**)&cache));
  iree_hal_resource_initialize(&b200_executable_cache_vtable, &cache->resource);
  cache->host_allocator = host_allocator;
  cache->device = device;
  *out_executable_cache = (iree_hal_executable_cache_t*)cache;
  return iree_ok_status();
}

static void b200_executable_cache_destroy(iree_hal_executable_cache_t* base_cache) {
  b200_executable_cache_t* cache = (b200_executable_cache_t*)base_cache;
  iree_allocator_free(cache->host_allocator, cache);
}

static bool b200_executable_cache_can_prepare_format(iree_hal_executable_cache_t* base_cache,
                                                     iree_hal_executable_caching_mode_t caching_mode,
                                                     iree_string_view_t executable_format) {
  return iree_string_view_equal(executable_format, iree_make_cstring_view(TB200_OPS_FORMAT_STRING));
}

// The blob names its own format in its first word; anything else is not ours.
static iree_status_t b200_executable_cache_infer_format(iree_hal_executable_cache_t* base_cache,
                                                        iree_hal_executable_caching_mode_t caching_mode,
                                                        iree_const_byte_span_t executable_data,
                                                        iree_host_size_t executable_format_capacity,
                                                        char* executable_format, iree_host_size_t* out_inferred_size) {
  uint32_t magic = 0;
  if (executable_data.data_length >= sizeof(tb200_ops_header_t)) memcpy(&magic, executable_data.data, sizeof(magic));
  if (magic != TB200_OPS_MAGIC) {
    return iree_make_status(IREE_STATUS_INCOMPATIBLE, "not a %s executable", TB200_OPS_FORMAT_STRING);
  }
  const iree_string_view_t format = iree_make_cstring_view(TB200_OPS_FORMAT_STRING);
  if (format.size >= executable_format_capacity) {
    return iree_make_status(IREE_STATUS_OUT_OF_RANGE, "executable format buffer too small");
  }
  memcpy(executable_format, format.data, format.size + 1);
  tb200_ops_header_t header;
  memcpy(&header, executable_data.data, sizeof(header));
  *out_inferred_size = (iree_host_size_t)header.total_bytes;
  return iree_ok_status();
}

static iree_status_t b200_executable_cache_prepare_executable(iree_hal_executable_cache_t* base_cache,
                                                              const iree_hal_executable_params_t* executable_params,
                                                              iree_hal_executable_t** out_executable) {
  b200_executable_cache_t* cache = (b200_executable_cache_t*)base_cache;
  if (!b200_executable_cache_can_prepare_format(base_cache, executable_params->caching_mode,
                                                executable_params->executable_format)) {
    return iree_make_status(IREE_STATUS_NOT_FOUND,
                            "no torq_b200 executable implementation registered for the given executable format '%.*s'",
                            (int)executable_params->executable_format.size, executable_params->executable_format.data);
  }
  return b200_executable_create(cache->device, cache->host_allocator, executable_params, out_executable);
}

static const iree_hal_executable_cache_vtable_t b200_executable_cache_vtable = {
    .destroy = b200_executable_cache_destroy,
    .infer_format = b200_executable_cache_infer_format,
    .can_prepare_format = b200_executable_cache_can_prepare_format,
    .prepare_executable = b200_executable_cache_prepare_executable,
};
