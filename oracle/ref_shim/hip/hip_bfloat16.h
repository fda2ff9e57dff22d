/* Test infrastructure: the LM-head file of the reference includes this header name. */
#pragma once
#include "hip_bf16.h"
