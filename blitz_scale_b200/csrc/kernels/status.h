// Status codes a kernel writes to its status word when a bounded wait gives up
// or an index check fails.  0 means success; the host maps the others to errors.
#pragma once
namespace blitz {
enum StatusCode : int {
  kStatusOk = 0,
  kStatusTimeoutProducer = 1,
  kStatusTimeoutMma = 2,
  kStatusTimeoutEpilogue = 3,
  kStatusTimeoutFlag = 4,
  kStatusBadIndex = 5,
  kStatusTooLarge = 6,
};
}  // namespace blitz
