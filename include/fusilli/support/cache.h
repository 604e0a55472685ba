// Forwarding header: keeps the reference's include path `fusilli/support/cache.h` working.
#pragma once
#include "../graph.h"
