# Block for the reference's iree_runtime_plugin.cmake, next to the one that enables "torq"
# (iree_runtime_plugin.cmake:9-16 of the reference). Enable with
#   -DIREE_EXTERNAL_HAL_DRIVERS="torq_b200"   (or "torq;torq_b200")
set(IREE_TORQ_ENABLE_TORQ_B200_DRIVER OFF)
if("torq_b200" IN_LIST IREE_EXTERNAL_HAL_DRIVERS)
  message(STATUS "Enabling the torq_b200 HAL driver (CUDA, sm_100a)")
  set(IREE_TORQ_ENABLE_TORQ_B200_DRIVER ON)
  add_subdirectory(${CMAKE_CURRENT_LIST_DIR}/runtime/driver_b200 TORQ_B200)
endif()
