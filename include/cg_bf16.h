/* cg_bf16.h: the reference keeps bf16 tensors and mixed precision in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_BF16_H
#define COGITO_COMPAT_CG_BF16_H
#include "cogito.h"
#endif
