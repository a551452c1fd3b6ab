/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/rotary_embedding/rotary_embedding.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
