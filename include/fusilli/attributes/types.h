// Forwarding header: keeps the reference's include path `fusilli/attributes/types.h` working.
#pragma once
#include "../types.h"
