// bf16 instances of the dA+dR kernel (a translation unit of their own: they compile side by side with the fp16 ones)
#include "prism_bwd_dadr_kernel.cuh"

namespace prism {
PRISM_DADR_DEFINE_PICKER(dadr_kernel_bf16, DT_BF16)
}  // namespace prism
