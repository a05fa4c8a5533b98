/* cg_speculative.h: the reference keeps samplers and speculative decoding in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_SPECULATIVE_H
#define COGITO_COMPAT_CG_SPECULATIVE_H
#include "cogito.h"
#endif
