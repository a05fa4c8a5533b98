/* cg_serialization.h: the reference keeps COG1 checkpoints in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_SERIALIZATION_H
#define COGITO_COMPAT_CG_SERIALIZATION_H
#include "cogito.h"
#endif
