// Glue between the public C header and the templated launchers: includes the header in
// "library build" mode (so 16-bit float pointers are the CUDA types) and provides the
// helpers that turn by-value scalar arguments into element values.
//
// Each family's .cu file is compiled once per dtype with -DMX_T=<suffix> and
// -DMX_TCLASS=<1 float | 2 unsigned | 3 signed | 4 bool>, which keeps every translation
// unit small enough to build in parallel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#define MAIDENX_CUDA_BUILD
#include "maidenx_cuda.h"

#include "common.cuh"

#define MX_CLASS_FLOAT 1
#define MX_CLASS_UINT 2
#define MX_CLASS_SINT 3
#define MX_CLASS_BOOL 4

namespace mx {
template <class T, class A>
inline T scalar_arg(A v) {
    return (T)v;
}
template <>
inline bf16 scalar_arg<bf16, uint16_t>(uint16_t v) {
    __nv_bfloat16_raw r;
    r.x = v;
    return bf16(r);
}
template <>
inline f16 scalar_arg<f16, uint16_t>(uint16_t v) {
    __half_raw r;
    r.x = v;
    return f16(r);
}
}  // namespace mx
