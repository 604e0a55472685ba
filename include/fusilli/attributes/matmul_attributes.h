// Forwarding header: keeps the reference's include path `fusilli/attributes/matmul_attributes.h` working.
#pragma once
#include "../attributes.h"
