/* cg_fusion.h: the reference keeps the fusion pass in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_FUSION_H
#define COGITO_COMPAT_CG_FUSION_H
#include "cogito.h"
#endif
