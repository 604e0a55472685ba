// Forwarding header: keeps the reference's include path `fusilli/node/conv_node.h` working.
#pragma once
#include "../nodes.h"
