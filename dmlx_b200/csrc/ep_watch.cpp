// Host-side watchdog for the collectives of the expert-parallel layer: waits for the work queued on a
// stream while polling the communicator's asynchronous error state, and aborts the communicator when
// an error shows up or the time limit passes (a peer that has gone leaves the collective waiting for
// ever; aborting it returns the GPU to the caller).  The three operations come in as callbacks, so the
// loop itself is plain C++ and is tested on the CPU with fakes.
#include <chrono>
#include <thread>

#include "dmlx_b200.h"

extern "C" int32_t b200_ep_watch(const b200_ep_watch_ops* ops, int32_t timeout_ms, int32_t poll_us) {
  const auto t0 = std::chrono::steady_clock::now();
  if (poll_us <= 0) poll_us = 100;
  for (;;) {
    if (ops->done(ops->ctx)) return B200_EP_WATCH_DONE;
    if (ops->async_error(ops->ctx) != 0) {
      ops->abort(ops->ctx);
      return B200_EP_WATCH_ERROR;
    }
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (timeout_ms >= 0 && ms >= timeout_ms) {
      ops->abort(ops->ctx);
      return B200_EP_WATCH_TIMEOUT;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
  }
}
