// Host-side state shared by the entry points of libattn_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// One status word per device, allocated on first use and kept until process
// exit.  Kernels record the id of a wait that ran out here; a non-zero word
// makes every later kernel of this library return at once, until
// attn_b200_last_device_status() has read (and thereby cleared) it.
int* device_status_word(int device);

}  // namespace b200
