// Shared includes and small helpers of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cusync_b200.h"
#include "../../include/cusync/cusync_defines.h"
#include "../../include/cusync/policy_eval.h"
#include "../../include/cusync/device-functions.h"
