/* cg_cuda.h: the reference keeps the device layer in a header of this name; here it is declared by cogito_cuda.h. */
#ifndef COGITO_COMPAT_CG_CUDA_H
#define COGITO_COMPAT_CG_CUDA_H
#include "cogito.h"
#include "cogito_cuda.h"
#endif
