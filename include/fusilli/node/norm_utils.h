// Forwarding header: keeps the reference's include path `fusilli/node/norm_utils.h` working.
#pragma once
#include "../nodes.h"
