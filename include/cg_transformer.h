/* cg_transformer.h: the reference keeps the transformer block in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_TRANSFORMER_H
#define COGITO_COMPAT_CG_TRANSFORMER_H
#include "cogito.h"
#endif
