// Registers the "torq_b200" driver factory with IREE's driver registry: the counterpart of
// runtime/driver/registration/driver_module.c:83-168 of the reference. There are no host
// executable loaders and no allocator flag here: device memory is HBM behind the C ABI.
// Uncompiled here (IREE's headers are absent from this tree).
#include "registration/driver_module.h"

#include "b200_hal.h"

static iree_status_t b200_factory_enumerate(void* self, iree_host_size_t* out_driver_info_count,
                                            const iree_hal_driver_info_t** out_driver_infos) {
  static const iree_hal_driver_info_t info = {
      .driver_name = IREE_SVL("torq_b200"),
      .full_name = IREE_SVL("Torq quantized layer ops on NVIDIA B200 (CUDA, sm_100a)"),
  };
  *out_driver_info_count = 1;
  *out_driver_infos = &info;
  return iree_ok_status();
}

static iree_status_t b200_factory_try_create(void* self, iree_string_view_t driver_name, iree_allocator_t host_allocator,
                                             iree_hal_driver_t** out_driver) {
  if (!iree_string_view_equal(driver_name, IREE_SV("torq_b200"))) {
    return iree_make_status(IREE_STATUS_UNAVAILABLE, "no driver '%.*s' is provided by this factory",
                            (int)driver_name.size, driver_name.data);
  }
  return iree_hal_torq_b200_driver_create(driver_name, host_allocator, out_driver);
}

IREE_API_EXPORT iree_status_t iree_hal_torq_b200_driver_module_register(iree_hal_driver_registry_t* registry) {
  static const iree_hal_driver_factory_t factory = {
      .self = NULL,
      .enumerate = b200_factory_enumerate,
      .try_create = b200_factory_try_create,
  };
  return iree_hal_driver_registry_register_factory(registry, &factory);
}
