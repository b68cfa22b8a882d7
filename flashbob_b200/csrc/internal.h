// Declarations shared by the translation units of libbob_sm100.so that are not part of the C ABI.
#pragma once

#include "../../include/bob_sm100.h"

namespace bob {

// Which kernels of the second backward to launch.
enum : int { kPartRow = 1, kPartCol = 2, kPartBoth = 3 };

// Body of the second backward.  `sticky` (nullable) is a device-visible word that a kernel also
// writes when a bounded wait runs out; `part` selects the kernels; `allow_split` lets long
// column-owned work items be divided between two CTAs, which needs the extra workspace that
// bob_sm100_workspace_bytes reports (callers with a fixed-size scratch pass false).
int bwd2_impl(const bob_sm100_geom* g, const void* q, const void* k, const void* v, const void* out,
              const float* lse, const float* delta, const float* pk, const void* dO, const void* dQ,
              const void* uQ, const void* uK, const void* uV, void* Qbar, void* Kbar, void* Vbar,
              void* dObar, void* workspace, void* stream, int* sticky, int part, bool allow_split);

// The per-device host-visible status word: its device address (create = true: page-locks it on first
// use; null if that failed) or its host address (create = false; null before first use).
int* sticky_word(int device, bool create);

// Bytes of the second backward's workspace without the area for divided work items.
size_t bwd2_workspace_bytes_unsplit(const bob_sm100_geom* g);

}  // namespace bob
