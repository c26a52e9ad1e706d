// reduce_by_key instantiations for unsigned long long values.
#include "abi_rbk.cuh"
namespace tb200_abi { TB200_RBK_INST(unsigned long long) }
