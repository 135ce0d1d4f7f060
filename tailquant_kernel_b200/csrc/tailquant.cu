// libtailquant.so is one translation unit: the kernel files share the device-side status
// word and the PTX wrappers, and none of them needs relocatable device code.
#include "tq_api.cu"
#include "tq_prologue_fast.cu"
#include "tq_prologue.cu"
#include "tq_gemm.cu"
#include "tq_gemm_tail.cu"
#include "tq_gemm_pair.cu"
#include "tq_tail.cu"
#include "tq_misc.cu"
#include "tq_decode.cu"
