/* cg_layers.h: the reference keeps layers in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_LAYERS_H
#define COGITO_COMPAT_CG_LAYERS_H
#include "cogito.h"
#endif
