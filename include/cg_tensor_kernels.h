/* cg_tensor_kernels.h: the reference keeps device tensor operations in a header of this name; here it is declared by cogito_cuda.h. */
#ifndef COGITO_COMPAT_CG_TENSOR_KERNELS_H
#define COGITO_COMPAT_CG_TENSOR_KERNELS_H
#include "cogito.h"
#include "cogito_cuda.h"
#endif
