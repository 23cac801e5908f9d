// Per-device error word written by kernels whose bounded waits or checked indices fail, and a host-side
// counter of kernel launches issued by this extension.
#pragma once
#include <stdint.h>

namespace pfb {
int* status_word();          // device pointer to the current device's status word (allocated on first use)
int read_status(bool reset); // synchronises the current stream; returns the status (0 = ok)
void set_wait_budget(double seconds);  // budget of each bounded device-side wait (<= 0 restores the default, 1 s)
void count_launch(int n = 1);
int64_t launch_count(bool reset);
}  // namespace pfb
