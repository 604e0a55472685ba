// Forwarding header: keeps the reference's include path `fusilli/graph/context.h` working.
#pragma once
#include "../tensor.h"
