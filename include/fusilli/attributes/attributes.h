// Forwarding header: keeps the reference's include path `fusilli/attributes/attributes.h` working.
#pragma once
#include "../attributes.h"
