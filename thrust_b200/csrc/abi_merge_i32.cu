// merge and merge sort instantiations for int32_t keys.
#include "abi_merge.cuh"
namespace tb200_abi { TB200_MERGE_INST(int32_t) }
