// Forwarding header: keeps the reference's include path `fusilli/attributes/layernorm_attributes.h` working.
#pragma once
#include "../attributes.h"
