// Forwarding header: keeps the reference's include path `fusilli/backend/handle.h` working.
#pragma once
#include "../backend.h"
