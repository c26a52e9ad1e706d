// merge and merge sort instantiations for uint32_t keys.
#include "abi_merge.cuh"
namespace tb200_abi { TB200_MERGE_INST(uint32_t) }
