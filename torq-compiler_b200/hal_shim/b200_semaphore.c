// Timeline semaphore of the torq_b200 HAL driver. The HAL surface of this driver stays synchronous like
// the reference's (work is complete when queue_execute returns, runtime/driver/torq_device.c:487-526), so
// a semaphore is a host-side counter: a mutex, a value, a failure status, and one notification that every
// signal posts. Slots as in runtime/driver/torq_semaphore.c (destroy, query, signal, fail, wait).
// Uncompiled here (IREE's headers are absent from this tree).
#include "b200_hal.h"
#include "iree/base/internal/synchronization.h"

typedef struct b200_semaphore_t {
  iree_hal_semaphore_t base;
  iree_allocator_t host_allocator;
  iree_slim_mutex_t mutex;
  iree_notification_t notification;
  uint64_t value;
  iree_status_t failure;  // ok until fail() is called
} b200_semaphore_t;

static const iree_hal_semaphore_vtable_t b200_semaphore_vtable;

bool iree_hal_torq_b200_semaphore_isa(iree_hal_semaphore_t* semaphore) {
  return iree_hal_resource_is(&semaphore->resource, &b200_semaphore_vtable);
}

iree_status_t iree_hal_torq_b200_semaphore_create(uint64_t initial_value, iree_allocator_t host_allocator,
                                                  iree_hal_semaphore_t** out_semaphore) {
  *out_semaphore = NULL;
  b200_semaphore_t* semaphore = NULL;
  IREE_RETURN_IF_ERROR(iree_allocator_malloc(host_allocator, sizeof(*semaphore), (void**)&semaphore));
  iree_hal_semaphore_initialize(&b200_semaphore_vtable, &semaphore->base);
  semaphore->host_allocator = host_allocator;
  iree_slim_mutex_initialize(&semaphore->mutex);
  iree_notification_initialize(&semaphore->notification);
  semaphore->value = initial_value;
  semaphore->failure = iree_ok_status();
  *out_semaphore = &semaphore->base;
  return iree_ok_status();
}

static void b200_semaphore_destroy(iree_hal_semaphore_t* base) {
  b200_semaphore_t* semaphore = (b200_semaphore_t*)base;
  iree_status_ignore(semaphore->failure);
  iree_notification_deinitialize(&semaphore->notification);
  iree_slim_mutex_deinitialize(&semaphore->mutex);
  iree_hal_semaphore_deinitialize(&semaphore->base);
  iree_allocator_free(semaphore->host_allocator, semaphore);
}

static iree_status_t b200_semaphore_query(iree_hal_semaphore_t* base, uint64_t* out_value) {
  b200_semaphore_t* semaphore = (b200_semaphore_t*)base;
  iree_slim_mutex_lock(&semaphore->mutex);
  *out_value = semaphore->value;
  iree_status_t status = *out_value >= IREE_HAL_SEMAPHORE_FAILURE_VALUE ? iree_status_clone(semaphore->failure) : iree_ok_status();
  iree_slim_mutex_unlock(&semaphore->mutex);
  return status;
}

static iree_status_t b200_semaphore_signal(iree_hal_semaphore_t* base, uint64_t new_value) {
  b200_semaphore_t* semaphore = (b200_semaphore_t*)base;
  iree_slim_mutex_lock(&semaphore->mutex);
  iree_status_t status = iree_ok_status();
  if (new_value <= semaphore->value) {
    status = iree_make_status(IREE_STATUS_OUT_OF_RANGE, "semaphore values must increase monotonically");
  } else {
    semaphore->value = new_value;
  }
  iree_slim_mutex_unlock(&semaphore->mutex);
  if (iree_status_is_ok(status)) {
    iree_hal_semaphore_notify(&semaphore->base, new_value, IREE_STATUS_OK);  // timepoints registered by other drivers
    iree_notification_post(&semaphore->notification, IREE_ALL_WAITERS);
  }
  return status;
}

static void b200_semaphore_fail(iree_hal_semaphore_t* base, iree_status_t status) {
  b200_semaphore_t* semaphore = (b200_semaphore_t*)base;
  const iree_status_code_t code = iree_status_code(status);
  iree_slim_mutex_lock(&semaphore->mutex);
  if (!iree_status_is_ok(semaphore->failure)) {  // the first failure is kept
    iree_slim_mutex_unlock(&semaphore->mutex);
    iree_status_ignore(status);
    return;
  }
  semaphore->value = IREE_HAL_SEMAPHORE_FAILURE_VALUE;
  semaphore->failure = status;
  iree_slim_mutex_unlock(&semaphore->mutex);
  iree_hal_semaphore_notify(&semaphore->base, IREE_HAL_SEMAPHORE_FAILURE_VALUE, code);
  iree_notification_post(&semaphore->notification, IREE_ALL_WAITERS);
}

typedef struct b200_wait_t {
  b200_semaphore_t* semaphore;
  uint64_t value;
} b200_wait_t;

static bool b200_semaphore_reached(b200_wait_t* wait) {
  iree_slim_mutex_lock(&wait->semaphore->mutex);
  const bool reached = wait->semaphore->value >= wait->value;  // a failed semaphore holds the failure value
  iree_slim_mutex_unlock(&wait->semaphore->mutex);
  return reached;
}

static iree_status_t b200_semaphore_wait(iree_hal_semaphore_t* base, uint64_t value, iree_timeout_t timeout,
                                         iree_hal_wait_flags_t flags) {
  b200_semaphore_t* semaphore = (b200_semaphore_t*)base;
  b200_wait_t wait = {semaphore, value};
  if (!b200_semaphore_reached(&wait)) {
    if (iree_timeout_is_immediate(timeout)) return iree_status_from_code(IREE_STATUS_DEADLINE_EXCEEDED);
    iree_notification_await(&semaphore->notification, (iree_condition_fn_t)b200_semaphore_reached, &wait, timeout);
  }
  iree_slim_mutex_lock(&semaphore->mutex);
  iree_status_t status = iree_ok_status();
  if (!iree_status_is_ok(semaphore->failure)) status = iree_status_from_code(IREE_STATUS_ABORTED);
  else if (semaphore->value < value) status = iree_status_from_code(IREE_STATUS_DEADLINE_EXCEEDED);
  iree_slim_mutex_unlock(&semaphore->mutex);
  return status;
}

// Every semaphore of the list in turn (wait-all), or a poll loop over the list (wait-any). Work of this
// driver is complete when its queue call returns, so these waits only ever block on other threads' signals.
iree_status_t iree_hal_torq_b200_semaphore_multi_wait(iree_hal_wait_mode_t wait_mode,
                                                      const iree_hal_semaphore_list_t semaphore_list,
                                                      iree_timeout_t timeout) {
  const iree_time_t deadline_ns = iree_timeout_as_deadline_ns(timeout);
  if (wait_mode == IREE_HAL_WAIT_MODE_ALL) {
    for (iree_host_size_t i = 0; i < semaphore_list.count; ++i) {
      IREE_RETURN_IF_ERROR(iree_hal_semaphore_wait(semaphore_list.semaphores[i], semaphore_list.payload_values[i],
                                                   iree_make_deadline(deadline_ns), IREE_HAL_WAIT_FLAG_DEFAULT));
    }
    return iree_ok_status();
  }
  for (;;) {
    for (iree_host_size_t i = 0; i < semaphore_list.count; ++i) {
      uint64_t value = 0;
      IREE_RETURN_IF_ERROR(iree_hal_semaphore_query(semaphore_list.semaphores[i], &value));
      if (value >= semaphore_list.payload_values[i]) return iree_ok_status();
    }
    if (iree_time_now() >= deadline_ns) return iree_status_from_code(IREE_STATUS_DEADLINE_EXCEEDED);
    iree_thread_yield();
  }
}

static const iree_hal_semaphore_vtable_t b200_semaphore_vtable = {
    .destroy = b200_semaphore_destroy,
    .query = b200_semaphore_query,
    .signal = b200_semaphore_signal,
    .fail = b200_semaphore_fail,
    .wait = b200_semaphore_wait,
};
