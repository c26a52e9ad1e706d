// reduce_by_key instantiations for int32_t values.
#include "abi_rbk.cuh"
namespace tb200_abi { TB200_RBK_INST(int32_t) }
