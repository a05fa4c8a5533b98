/* cg_quantize.h: the reference keeps quantisation and the INT4 KV cache in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_QUANTIZE_H
#define COGITO_COMPAT_CG_QUANTIZE_H
#include "cogito.h"
#endif
