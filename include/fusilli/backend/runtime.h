// Forwarding header: keeps the reference's include path `fusilli/backend/runtime.h` working.
#pragma once
#include "../graph.h"
