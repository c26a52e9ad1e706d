// reduce_by_key instantiations for long long values.
#include "abi_rbk.cuh"
namespace tb200_abi { TB200_RBK_INST(long long) }
