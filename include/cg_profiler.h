/* cg_profiler.h: the reference keeps the profiler in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_PROFILER_H
#define COGITO_COMPAT_CG_PROFILER_H
#include "cogito.h"
#endif
