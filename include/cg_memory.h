/* cg_memory.h: the reference keeps pool, buddy allocator, planner in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_MEMORY_H
#define COGITO_COMPAT_CG_MEMORY_H
#include "cogito.h"
#endif
