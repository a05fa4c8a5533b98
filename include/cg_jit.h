/* cg_jit.h: the reference keeps the JIT IR in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_JIT_H
#define COGITO_COMPAT_CG_JIT_H
#include "cogito.h"
#endif
