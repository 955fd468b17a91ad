// Internal declarations of the torq_b200 HAL driver: one IREE object per C-ABI object.
// Uncompiled here (IREE's headers are absent from this tree); see README.md.
#ifndef TORQ_B200_HAL_SHIM_B200_HAL_H_
#define TORQ_B200_HAL_SHIM_B200_HAL_H_

#include "iree/base/api.h"
#include "iree/hal/api.h"
#include "torq_b200.h"
#include "torq_b200_ops.h"

#ifdef __cplusplus
extern "C" {
#endif

// tb200 status numbers are iree_status_code_t values (include/torq_b200.h), so a failed call
// becomes an iree_status_t with the same code and the library's message.
iree_status_t iree_hal_torq_b200_status(int tb200_status, tb200_device_t* device, const char* what);
#define B200_RETURN_IF_ERROR(device, expr)                                   \
  do {                                                                       \
    const int b200_status_ = (expr);                                         \
    if (b200_status_ != TB200_OK)                                            \
      return iree_hal_torq_b200_status(b200_status_, (device), #expr);       \
  } while (0)

//===-- driver ---------------------------------------------------------------
iree_status_t iree_hal_torq_b200_driver_create(iree_string_view_t identifier, iree_allocator_t host_allocator,
                                               iree_hal_driver_t** out_driver);

//===-- device ---------------------------------------------------------------
iree_status_t iree_hal_torq_b200_device_create(iree_string_view_t identifier, int cuda_ordinal,
                                               iree_allocator_t host_allocator, iree_hal_device_t** out_device);
// The C-ABI device behind a HAL device of this driver.
tb200_device_t* iree_hal_torq_b200_device_handle(iree_hal_device_t* device);

//===-- allocator and buffers ------------------------------------------------
iree_status_t iree_hal_torq_b200_allocator_create(tb200_device_t* device, iree_allocator_t host_allocator,
                                                  iree_hal_allocator_t** out_allocator);
// The C-ABI buffer behind a HAL buffer allocated by this driver (NULL for foreign buffers).
tb200_buffer_t* iree_hal_torq_b200_buffer_handle(iree_hal_buffer_t* buffer);

//===-- command buffer -------------------------------------------------------
iree_status_t iree_hal_torq_b200_command_buffer_create(iree_hal_allocator_t* device_allocator, tb200_device_t* device,
                                                       iree_hal_command_buffer_mode_t mode,
                                                       iree_hal_command_category_t command_categories,
                                                       iree_hal_queue_affinity_t queue_affinity,
                                                       iree_host_size_t binding_capacity, iree_allocator_t host_allocator,
                                                       iree_hal_command_buffer_t** out_command_buffer);
bool iree_hal_torq_b200_command_buffer_isa(iree_hal_command_buffer_t* command_buffer);

//===-- executables ----------------------------------------------------------
iree_status_t iree_hal_torq_b200_executable_cache_create(tb200_device_t* device, iree_string_view_t identifier,
                                                         iree_allocator_t host_allocator,
                                                         iree_hal_executable_cache_t** out_executable_cache);
// The C-ABI executable behind a HAL executable of this driver.
tb200_executable_t* iree_hal_torq_b200_executable_handle(iree_hal_executable_t* executable);

//===-- semaphores -----------------------------------------------------------
iree_status_t iree_hal_torq_b200_semaphore_create(uint64_t initial_value, iree_allocator_t host_allocator,
                                                  iree_hal_semaphore_t** out_semaphore);
bool iree_hal_torq_b200_semaphore_isa(iree_hal_semaphore_t* semaphore);
iree_status_t iree_hal_torq_b200_semaphore_multi_wait(iree_hal_wait_mode_t wait_mode,
                                                      const iree_hal_semaphore_list_t semaphore_list,
                                                      iree_timeout_t timeout);

#ifdef __cplusplus
}
#endif
#endif  // TORQ_B200_HAL_SHIM_B200_HAL_H_
