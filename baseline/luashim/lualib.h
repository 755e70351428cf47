#ifndef SHIM_LUALIB_H
#define SHIM_LUALIB_H
#include "lua.h"
#endif
