// Drop-in path of the reference header of the same name; see cpu_ops/b200/epilogue_types.h.
#pragma once
#include "cpu_ops/b200/epilogue_types.h"
