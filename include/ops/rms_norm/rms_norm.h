/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/rms_norm/rms_norm.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
