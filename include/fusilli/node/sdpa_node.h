// Forwarding header: keeps the reference's include path `fusilli/node/sdpa_node.h` working.
#pragma once
#include "../nodes.h"
