// Build-only forced include for compiling the reference against the CUTLASS 4.x
// headers found on this image (the reference pins CUTLASS v3.3.0, which is not
// available offline).  CUTLASS 4.x moved this trait into arch::detail; in v3.3.0
// it is true only for the FastF32 math operators, never for the fp16 path.
#pragma once
#include "cutlass/arch/mma.h"
namespace cutlass {
namespace arch {
template <typename MathOp>
struct UseStagedAccumulation { static bool const value = false; };
}  // namespace arch
}  // namespace cutlass
