// Entry symbol of the torq_b200 HAL driver; same signature as the reference's
// iree_hal_torq_driver_module_register (runtime/driver/registration/driver_module.h:16-17).
#ifndef TORQ_B200_HAL_SHIM_REGISTRATION_DRIVER_MODULE_H_
#define TORQ_B200_HAL_SHIM_REGISTRATION_DRIVER_MODULE_H_

#include "iree/base/api.h"
#include "iree/hal/api.h"

#ifdef __cplusplus
extern "C" {
#endif

IREE_API_EXPORT iree_status_t iree_hal_torq_b200_driver_module_register(iree_hal_driver_registry_t* registry);

#ifdef __cplusplus
}
#endif
#endif  // TORQ_B200_HAL_SHIM_REGISTRATION_DRIVER_MODULE_H_
