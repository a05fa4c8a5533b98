/* cg_tensor.h: the reference keeps tensors and autograd in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_TENSOR_H
#define COGITO_COMPAT_CG_TENSOR_H
#include "cogito.h"
#endif
