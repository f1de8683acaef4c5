// Elastic-style entry points of the C ABI (include/mcep.h): flat receive layout,
// one copy of a token per destination rank.
#include "ep_elastic.cuh"
#include "ep_runtime_internal.h"

namespace mcep {

void elastic_release(mcep_buffer*) {}

}  // namespace mcep
