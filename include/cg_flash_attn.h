/* cg_flash_attn.h: the reference keeps flash attention, RoPE, ALiBi in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_FLASH_ATTN_H
#define COGITO_COMPAT_CG_FLASH_ATTN_H
#include "cogito.h"
#endif
