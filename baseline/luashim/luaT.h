#ifndef SHIM_LUAT_H
#define SHIM_LUAT_H
#include "lua.h"
void* luaT_checkudata(lua_State* L, int idx, const char* tname);
#endif
