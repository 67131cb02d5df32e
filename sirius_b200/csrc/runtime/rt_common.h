// Shared bits of the host-side runtime sources.
#pragma once
#include "../common.cuh"

namespace srt {
std::string default_shm_prefix();  // "colserve_shm_<user>_p<SIRIUS_PORT>" (common/util.h:113-132)
}
