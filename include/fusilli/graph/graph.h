// Forwarding header: keeps the reference's include path `fusilli/graph/graph.h` working.
#pragma once
#include "../graph.h"
