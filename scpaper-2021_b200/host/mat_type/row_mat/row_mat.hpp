// row_mat under the reference's own include path (mat_type/row_mat/row_mat.hpp); every weight container of the
// path is defined in mat_type/mat_type.h.
#pragma once
#include "../mat_type.h"
