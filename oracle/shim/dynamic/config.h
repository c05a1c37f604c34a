/* Stand-in for training/training_dynamic/config.h when the reference's cpu_ops.h is
 * compiled on Linux.  TEST INFRASTRUCTURE ONLY.
 * Supplies the AdamState layout (config.h:46) and the Accelerate calls. */
#pragma once
#include "../accelerate_shim.h"
typedef struct { float *m, *v; size_t n; } AdamState;
