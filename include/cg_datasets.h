/* cg_datasets.h: the reference keeps datasets and iterators in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_DATASETS_H
#define COGITO_COMPAT_CG_DATASETS_H
#include "cogito.h"
#endif
