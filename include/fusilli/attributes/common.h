// Forwarding header: keeps the reference's include path `fusilli/attributes/common.h` working.
#pragma once
#include "../attributes.h"
