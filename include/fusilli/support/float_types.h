// Forwarding header: keeps the reference's include path `fusilli/support/float_types.h` working.
#pragma once
#include "../types.h"
