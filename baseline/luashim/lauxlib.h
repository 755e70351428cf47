#ifndef SHIM_LAUXLIB_H
#define SHIM_LAUXLIB_H
#include <stdio.h>
#include "lua.h"

typedef struct luaL_Reg {
  const char* name;
  lua_CFunction func;
} luaL_Reg;
#define luaL_reg luaL_Reg

int luaL_checkint(lua_State* L, int idx);
const char* luaL_checkstring(lua_State* L, int idx);
void luaL_getmetatable(lua_State* L, const char* tname);
int luaL_newmetatable(lua_State* L, const char* tname);
void luaL_register(lua_State* L, const char* libname, const luaL_Reg* l);

#endif
