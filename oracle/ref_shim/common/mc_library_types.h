// Value-type enum of the MetaX SDK: the mcSparse tree carries its own copy for non-MACA
// builds. That copy also declares libraryPropertyType, which the CUDA runtime headers already
// define, so those names are moved out of the way while it is read.
#pragma once
#define libraryPropertyType_t mcsp_ref_libraryPropertyType_t
#define libraryPropertyType mcsp_ref_libraryPropertyType
#define MAJOR_VERSION MCSP_REF_MAJOR_VERSION
#define MINOR_VERSION MCSP_REF_MINOR_VERSION
#define PATCH_LEVEL MCSP_REF_PATCH_LEVEL
#include "common/internal/mcsp_datatype.h"
#undef libraryPropertyType_t
#undef libraryPropertyType
#undef MAJOR_VERSION
#undef MINOR_VERSION
#undef PATCH_LEVEL
