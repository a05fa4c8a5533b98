/* cg_symbolic.h: the reference keeps symbolic shapes in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_SYMBOLIC_H
#define COGITO_COMPAT_CG_SYMBOLIC_H
#include "cogito.h"
#endif
