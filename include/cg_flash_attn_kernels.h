/* cg_flash_attn_kernels.h: the reference keeps device attention in a header of this name; here it is declared by cogito_cuda.h. */
#ifndef COGITO_COMPAT_CG_FLASH_ATTN_KERNELS_H
#define COGITO_COMPAT_CG_FLASH_ATTN_KERNELS_H
#include "cogito.h"
#include "cogito_cuda.h"
#endif
