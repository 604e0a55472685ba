// Forwarding header: keeps the reference's include path `fusilli/attributes/pointwise_attributes.h` working.
#pragma once
#include "../attributes.h"
