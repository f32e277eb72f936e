// One error word per device, written by kernels whose bounded waits give up
// (0 = ok, otherwise a code naming the wait site).  Allocated on first use.
#pragma once
#include "common.h"

namespace rt {
int* device_error_word();
// Synchronises the device, reads and clears the word.
rt_status check_device_error(const char* what);
}  // namespace rt
