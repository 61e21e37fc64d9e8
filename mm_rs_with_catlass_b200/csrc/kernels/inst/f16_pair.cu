// Instantiates the fused kernel for one operand kind and CTA flavour (see kernel_inst.cuh).
#include "catcoc/kernel_inst.cuh"

CATCOC_DEFINE_UNIT_4(f16_pair, catcoc::KIND_F16, true)
