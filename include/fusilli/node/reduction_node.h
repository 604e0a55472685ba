// Forwarding header: keeps the reference's include path `fusilli/node/reduction_node.h` working.
#pragma once
#include "../nodes.h"
