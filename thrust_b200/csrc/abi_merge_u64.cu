// merge and merge sort instantiations for unsigned long long keys.
#include "abi_merge.cuh"
namespace tb200_abi { TB200_MERGE_INST(unsigned long long) }
