/* Minimal stand-in for the Lua 5.1 C API: just enough surface for a C extension module that
 * registers functions, reads three kinds of arguments (integer, string, userdata) and creates one
 * userdata with a metatable.  There is no interpreter behind it: "the stack" is the argument list
 * of the call in progress, filled in by the host program (see ref_host.c). */
#ifndef SHIM_LUA_H
#define SHIM_LUA_H
#include <stddef.h>

typedef struct lua_State lua_State;
typedef int (*lua_CFunction)(lua_State* L);

void* lua_newuserdata(lua_State* L, size_t size);
int lua_setmetatable(lua_State* L, int idx);
void* lua_touserdata(lua_State* L, int idx);
void lua_pushvalue(lua_State* L, int idx);
void lua_setfield(lua_State* L, int idx, const char* key);

#endif
