/* Stand-in for training/stories_config.h when the reference's stories_cpu_ops.h is
 * compiled on Linux.  TEST INFRASTRUCTURE ONLY.
 * Supplies what the operator header needs from the real config: the AdamState layout
 * (stories_config.h:56-59), the VOCAB bound used by embed_lookup/embed_backward
 * (stories_config.h:24; made a run-time variable so one build serves several vocab sizes)
 * and the Accelerate calls (through accelerate_shim.h). */
#pragma once
#include "../accelerate_shim.h"
typedef struct { float *m, *v; size_t n; } AdamState;
extern int g_ref_vocab;
#define VOCAB g_ref_vocab
