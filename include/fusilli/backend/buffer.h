// Forwarding header: keeps the reference's include path `fusilli/backend/buffer.h` working.
#pragma once
#include "../backend.h"
