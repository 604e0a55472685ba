// Forwarding header: keeps the reference's include path `fusilli/backend/backend.h` working.
#pragma once
#include "../backend.h"
