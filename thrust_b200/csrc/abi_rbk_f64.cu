// reduce_by_key instantiations for double values.
#include "abi_rbk.cuh"
namespace tb200_abi { TB200_RBK_INST(double) }
