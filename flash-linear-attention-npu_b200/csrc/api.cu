// Library-level entry points.
#include "fla_b200_internal.h"

extern "C" FLA_API int fla_b200_version(void) { return 100; }
