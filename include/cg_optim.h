/* cg_optim.h: the reference keeps optimizers in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_OPTIM_H
#define COGITO_COMPAT_CG_OPTIM_H
#include "cogito.h"
#endif
