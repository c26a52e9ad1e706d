// reduce_by_key instantiations for uint32_t values.
#include "abi_rbk.cuh"
namespace tb200_abi { TB200_RBK_INST(uint32_t) }
