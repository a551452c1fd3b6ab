/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/random_sample/random_sample.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
