// Forwarding header: keeps the reference's include path `fusilli/attributes/conv_attributes.h` working.
#pragma once
#include "../attributes.h"
