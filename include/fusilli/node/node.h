// Forwarding header: keeps the reference's include path `fusilli/node/node.h` working.
#pragma once
#include "../nodes.h"
