// Forwarding header: keeps the reference's include path `fusilli/support/logging.h` working.
#pragma once
#include "../error.h"
