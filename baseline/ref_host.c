/* Host program for the unmodified reference module.
 *
 * The reference (src/sharedtensor.c of Hello1024/shared-tensor) is a Lua 5.1 extension for Torch7.
 * Neither Lua nor Torch7 is available, so this file plays the interpreter: it includes the
 * reference source verbatim (copied next to the build output, never edited), lets
 * luaopen_sharedtensor() register the module's functions, remembers them by name, and exposes
 * three plain C entry points that call them exactly as Lua would: through the registered
 * lua_CFunction with the arguments on the (emulated) stack.
 */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "lua.h"
#include "lauxlib.h"
#include "TH/THTensor.h"
#include "luaT.h"

/* ---- the emulated interpreter state: arguments of the call in progress ---- */
#define MAX_ARGS 4
enum { ARG_NONE, ARG_INT, ARG_STR, ARG_TENSOR, ARG_UDATA };
struct lua_State {
  int kind[MAX_ARGS + 1];
  long ival[MAX_ARGS + 1];
  const char* sval[MAX_ARGS + 1];
  void* pval[MAX_ARGS + 1];
  void* last_userdata; /* result of lua_newuserdata in this call */
};

static struct lua_State g_state;
static lua_CFunction fn_createOrFetch, fn_copyToTensor, fn_addFromTensor, fn_gc;

void* lua_newuserdata(lua_State* L, size_t size) {
  L->last_userdata = malloc(size);
  return L->last_userdata;
}
int lua_setmetatable(lua_State* L, int idx) { (void)L; (void)idx; return 1; }
void* lua_touserdata(lua_State* L, int idx) { return L->kind[idx] == ARG_UDATA ? L->pval[idx] : NULL; }
void lua_pushvalue(lua_State* L, int idx) { (void)L; (void)idx; }
void lua_setfield(lua_State* L, int idx, const char* key) { (void)L; (void)idx; (void)key; }

int luaL_checkint(lua_State* L, int idx) {
  if (L->kind[idx] != ARG_INT) { fprintf(stderr, "ref_host: argument %d is not an integer\n", idx); abort(); }
  return (int)L->ival[idx];
}
const char* luaL_checkstring(lua_State* L, int idx) {
  if (L->kind[idx] != ARG_STR) { fprintf(stderr, "ref_host: argument %d is not a string\n", idx); abort(); }
  return L->sval[idx];
}
void* luaT_checkudata(lua_State* L, int idx, const char* tname) {
  if (L->kind[idx] != ARG_TENSOR || strcmp(tname, "torch.FloatTensor") != 0) {
    fprintf(stderr, "ref_host: argument %d is not a %s\n", idx, tname);
    abort();
  }
  return L->pval[idx];
}
void luaL_getmetatable(lua_State* L, const char* tname) { (void)L; (void)tname; }
int luaL_newmetatable(lua_State* L, const char* tname) { (void)L; (void)tname; return 1; }
void luaL_register(lua_State* L, const char* libname, const luaL_Reg* l) {
  (void)L; (void)libname;
  for (; l->name; l++) {
    if (!strcmp(l->name, "createOrFetch")) fn_createOrFetch = l->func;
    else if (!strcmp(l->name, "copyToTensor")) fn_copyToTensor = l->func;
    else if (!strcmp(l->name, "addFromTensor")) fn_addFromTensor = l->func;
    else if (!strcmp(l->name, "__gc")) fn_gc = l->func;
  }
}
void THError(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  fprintf(stderr, "THError: ");
  vfprintf(stderr, fmt, ap);
  fprintf(stderr, "\n");
  va_end(ap);
  abort();
}

/* ---- the reference, verbatim ---- */
#include "sharedtensor.c"

/* ---- entry points for the host language (ctypes) ---- */
static void clear_args(void) { memset(&g_state, 0, sizeof(g_state)); }

__attribute__((visibility("default"))) int ref_open(void) {
  luaopen_sharedtensor(&g_state);
  return fn_createOrFetch && fn_copyToTensor && fn_addFromTensor ? 0 : -1;
}

/* sharedtensor.createOrFetch(host, port, tensor) -> userdata */
__attribute__((visibility("default"))) void* ref_createOrFetch(const char* host, int port, float* data, long n) {
  THFloatTensor t = {data, n};
  clear_args();
  g_state.kind[1] = ARG_STR;    g_state.sval[1] = host;
  g_state.kind[2] = ARG_INT;    g_state.ival[2] = port;
  g_state.kind[3] = ARG_TENSOR; g_state.pval[3] = &t;
  fn_createOrFetch(&g_state);
  return g_state.last_userdata;
}

/* z:copyToTensor(tensor) */
__attribute__((visibility("default"))) void ref_copyToTensor(void* z, float* data, long n) {
  THFloatTensor t = {data, n};
  clear_args();
  g_state.kind[1] = ARG_UDATA;  g_state.pval[1] = z;
  g_state.kind[2] = ARG_TENSOR; g_state.pval[2] = &t;
  fn_copyToTensor(&g_state);
}

/* z:addFromTensor(tensor) */
__attribute__((visibility("default"))) void ref_addFromTensor(void* z, float* data, long n) {
  THFloatTensor t = {data, n};
  clear_args();
  g_state.kind[1] = ARG_UDATA;  g_state.pval[1] = z;
  g_state.kind[2] = ARG_TENSOR; g_state.pval[2] = &t;
  fn_addFromTensor(&g_state);
}
