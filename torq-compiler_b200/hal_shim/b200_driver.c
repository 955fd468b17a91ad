// iree_hal_driver_t of the torq_b200 backend: enumerates the sm_100 GPUs of the node and creates one
// HAL device per CUDA ordinal. Slots as in runtime/driver/torq_driver.c:151-157 of the reference.
// Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"

#define B200_MAX_DEVICES 16

typedef struct b200_driver_t {
  iree_hal_resource_t resource;
  iree_allocator_t host_allocator;
  iree_string_view_t identifier;  // storage follows the struct
} b200_driver_t;

static const iree_hal_driver_vtable_t b200_driver_vtable;

iree_status_t iree_hal_torq_b200_status(int tb200_status, tb200_device_t* device, const char* what) {
  if (tb200_status == TB200_OK) return iree_ok_status();
  const char* message = device ? tb200_last_error(device) : "";
  return iree_make_status((iree_status_code_t)tb200_status, "%s: %s%s%s", what, tb200_status_string(tb200_status),
                          message[0] ? ": " : "", message);
}

iree_status_t iree_hal_torq_b200_driver_create(iree_string_view_t identifier, iree_allocator_t host_allocator,
                                               iree_hal_driver_t** out_driver) {
  IREE_ASSERT_ARGUMENT(out_driver);
  *out_driver = NULL;
  b200_driver_t* driver = NULL;
  const iree_host_size_t total = sizeof(*driver) + identifier.size;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, total, (void**)&driver));
  iree_hal_resource_initialize(&b200_driver_vtable, &driver->resource);
  driver->host_allocator = host_allocator;
  iree_string_view_append_to_buffer(identifier, &driver->identifier, (char*)driver + sizeof(*driver));
  *out_driver = (iree_hal_driver_t*)driver;
  return iree_ok_status();
}

static void b200_driver_destroy(iree_hal_driver_t* base_driver) {
  b200_driver_t* driver = (b200_driver_t*)base_driver;
  iree_allocator_free(driver->host_allocator, driver);
}

// A device is offered for every ordinal the C ABI can open (an sm_100 GPU); the probe opens and
// closes it, which costs a stream pair and is done once per enumeration.
static iree_status_t b200_driver_query_available_devices(iree_hal_driver_t* base_driver, iree_allocator_t host_allocator,
                                                         iree_host_size_t* out_device_info_count,
                                                         iree_hal_device_info_t** out_device_infos) {
  int ordinals[B200_MAX_DEVICES];
  iree_host_size_t count = 0;
  for (int ordinal = 0; ordinal < B200_MAX_DEVICES; ++ordinal) {
    tb200_device_t* probe = NULL;
    const int status = tb200_device_create(ordinal, &probe);
    if (status == TB200_NOT_FOUND) break;  // beyond the last GPU
    if (status != TB200_OK) continue;      // a GPU of another architecture
    tb200_device_destroy(probe);
    ordinals[count++] = ordinal;
  }
  iree_hal_device_info_t* infos = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, (count ? count : 1) * sizeof(*infos), (void**)&infos));
  for (iree_host_size_t i = 0; i < count; ++i) {
    infos[i].device_id = (iree_hal_device_id_t)ordinals[i];
    infos[i].path = iree_string_view_empty();
    infos[i].name = IREE_SV("NVIDIA B200 (sm_100a)");
  }
  *out_device_info_count = count;
  *out_device_infos = infos;
  return iree_ok_status();
}

static iree_status_t b200_driver_dump_device_info(iree_hal_driver_t* base_driver, iree_hal_device_id_t device_id,
                                                  iree_string_builder_t* builder) {
  return iree_string_builder_append_format(builder, "torq_b200 device %d: executable format '%s', ops version %u\n",
                                           (int)device_id, TB200_OPS_FORMAT_STRING, (unsigned)TB200_OPS_VERSION);
}

static iree_status_t b200_driver_create_device_by_id(iree_hal_driver_t* base_driver, iree_hal_device_id_t device_id,
                                                     iree_host_size_t param_count, const iree_string_pair_t* params,
                                                     iree_allocator_t host_allocator, iree_hal_device_t** out_device) {
  b200_driver_t* driver = (b200_driver_t*)base_driver;
  const int ordinal = device_id == IREE_HAL_DEVICE_ID_DEFAULT ? 0 : (int)device_id;
  return iree_hal_torq_b200_device_create(driver->identifier, ordinal, host_allocator, out_device);
}

// --device=torq_b200://<ordinal>; an empty path is the default device (ordinal 0).
static iree_status_t b200_driver_create_device_by_path(iree_hal_driver_t* base_driver, iree_string_view_t driver_name,
                                                       iree_string_view_t device_path, iree_host_size_t param_count,
                                                       const iree_string_pair_t* params, iree_allocator_t host_allocator,
                                                       iree_hal_device_t** out_device) {
  int32_t ordinal = 0;
  if (!iree_string_view_is_empty(device_path) && !iree_string_view_atoi_int32(device_path, &ordinal)) {
    return iree_make_status(IREE_STATUS_NOT_FOUND, "device path '%.*s' is not a CUDA ordinal", (int)device_path.size,
                            device_path.data);
  }
  return b200_driver_create_device_by_id(base_driver, (iree_hal_device_id_t)ordinal, param_count, params, host_allocator,
                                         out_device);
}

static const iree_hal_driver_vtable_t b200_driver_vtable = {
    .destroy = b200_driver_destroy,
    .query_available_devices = b200_driver_query_available_devices,
    .dump_device_info = b200_driver_dump_device_info,
    .create_device_by_id = b200_driver_create_device_by_id,
    .create_device_by_path = b200_driver_create_device_by_path,
};
