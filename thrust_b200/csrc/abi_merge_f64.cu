// merge and merge sort instantiations for double keys.
#include "abi_merge.cuh"
namespace tb200_abi { TB200_MERGE_INST(double) }
