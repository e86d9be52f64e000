// Device-side status words shared by all kernels of the library (one
// translation unit, so a plain definition is enough). See wsl_poll_status().
#pragma once
namespace wsl {
__device__ int g_wsl_status[4];
int device_check();      // WSL_OK when the current device is sm_100
int device_sm_count();   // valid after device_check() returned WSL_OK
}  // namespace wsl
