/* cg_grad_check.h: the reference keeps the gradient checker in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_GRAD_CHECK_H
#define COGITO_COMPAT_CG_GRAD_CHECK_H
#include "cogito.h"
#endif
