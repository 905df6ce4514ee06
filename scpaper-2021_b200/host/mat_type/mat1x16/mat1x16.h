// mat1x16 under the reference's own include path (mat_type/mat1x16/mat1x16.h); every weight container of the
// path is defined in mat_type/mat_type.h.
#pragma once
#include "../mat_type.h"
