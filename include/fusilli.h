// Umbrella header of the Fusilli front end on the B200 backend: the include path existing
// Fusilli programs use (`#include <fusilli.h>`), same public names as the reference's
// include/fusilli.h.
#ifndef FUSILLI_H
#define FUSILLI_H

#include "fusilli/error.h"
#include "fusilli/types.h"
#include "fusilli/tensor.h"
#include "fusilli/attributes.h"
#include "fusilli/nodes.h"
#include "fusilli/backend.h"
#include "fusilli/graph.h"
#include "fusilli/comm.h"

#endif // FUSILLI_H
