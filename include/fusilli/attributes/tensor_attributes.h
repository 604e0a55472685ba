// Forwarding header: keeps the reference's include path `fusilli/attributes/tensor_attributes.h` working.
#pragma once
#include "../tensor.h"
