// Forwarding header: keeps the reference's include path `fusilli/attributes/sdpa_attributes.h` working.
#pragma once
#include "../attributes.h"
