// forwards to the shim of the reference header of this name
#pragma once
#include "jittor_shim.h"
