/* cg_arena.h: the reference keeps arenas in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_ARENA_H
#define COGITO_COMPAT_CG_ARENA_H
#include "cogito.h"
#endif
