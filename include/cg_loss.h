/* cg_loss.h: the reference keeps losses in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_LOSS_H
#define COGITO_COMPAT_CG_LOSS_H
#include "cogito.h"
#endif
