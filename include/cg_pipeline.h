/* cg_pipeline.h: the reference keeps pipeline / tensor / 3-D parallel types and schedules in a header of this name; here everything is declared by cogito.h. */
#ifndef COGITO_COMPAT_CG_PIPELINE_H
#define COGITO_COMPAT_CG_PIPELINE_H
#include "cogito.h"
#endif
