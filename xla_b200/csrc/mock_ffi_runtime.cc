// A small stand-in for the XLA side of the FFI, for tests and benchmarks in environments where
// XLA itself cannot be built.  It implements the `XLA_FFI_Api` function table with the real
// structs of xla/ffi/api/c_api.h and drives a handler the way XLA's CustomCallThunk does
// (xla/backends/gpu/runtime/custom_call_thunk.cc:179-240, 451-560):
//   registration: look at the bundle, query the execute handler's metadata (API version,
//                 traits) and refuse unsupported versions (xla/ffi/ffi_registry.cc:47-65, 87-158);
//   per call site: `instantiate` once with null buffer data, then prepare -> initialize ->
//                 execute with the real device pointers.
// Nothing here is on the product path: a real XLA process supplies its own XLA_FFI_Api.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "xla/ffi/api/c_api.h"

#define MOCK_EXPORT extern "C" __attribute__((visibility("default")))

struct XLA_FFI_Error {
  XLA_FFI_Error_Code code;
  std::string message;
};

// What a handler sees as its opaque execution context.
struct XLA_FFI_InvokeContext {
  void* stream = nullptr;
  int32_t device_ordinal = 0;
  int64_t run_id = 1;
  std::map<int, std::pair<int64_t, void*>>* state = nullptr;   // stage -> (type id, state)
};

namespace {

struct Registration {
  XLA_FFI_Handler_Bundle bundle{};
  XLA_FFI_Handler_Traits traits = 0;
  XLA_FFI_Metadata metadata{};
};

std::mutex g_mu;
std::map<std::string, Registration>& Registry() {
  static auto* r = new std::map<std::string, Registration>();
  return *r;
}
int64_t g_next_type_id = 1;

XLA_FFI_Error* NewError(XLA_FFI_Error_Code code, std::string msg) { return new XLA_FFI_Error{code, std::move(msg)}; }

// ---- XLA_FFI_Api entries -------------------------------------------------------------------
XLA_FFI_Error* ErrorCreate(XLA_FFI_Error_Create_Args* a) { return NewError(a->errc, a->message ? a->message : ""); }
void ErrorGetDetails(XLA_FFI_Error_GetDetails_Args* a) {
  a->message = a->error->message.c_str();
  a->errc = a->error->code;
}
void ErrorDestroy(XLA_FFI_Error_Destroy_Args* a) { delete a->error; }

const XLA_FFI_Api* Api();

XLA_FFI_Error* HandlerRegister(XLA_FFI_Handler_Register_Args* a) {
  const std::string name(a->name.ptr, a->name.len);
  const std::string platform(a->platform.ptr, a->platform.len);
  if (a->bundle.execute == nullptr) return NewError(XLA_FFI_Error_Code_INVALID_ARGUMENT, "execute handler is required");
  // Ask the execute handler for its metadata through the metadata extension.
  XLA_FFI_Metadata metadata{};
  metadata.struct_size = XLA_FFI_Metadata_STRUCT_SIZE;
  XLA_FFI_Metadata_Extension ext{};
  ext.extension_base.struct_size = XLA_FFI_Metadata_Extension_STRUCT_SIZE;
  ext.extension_base.type = XLA_FFI_Extension_Metadata;
  ext.extension_base.next = nullptr;
  ext.metadata = &metadata;
  XLA_FFI_CallFrame frame{};
  frame.struct_size = XLA_FFI_CallFrame_STRUCT_SIZE;
  frame.extension_start = &ext.extension_base;
  frame.api = Api();
  if (XLA_FFI_Error* e = a->bundle.execute(&frame)) return e;
  const int major = metadata.api_version.major_version, minor = metadata.api_version.minor_version;
  if (major != XLA_FFI_API_MAJOR || minor < 1 || minor > XLA_FFI_API_MINOR)
    return NewError(XLA_FFI_Error_Code_INVALID_ARGUMENT,
                    "FFI handler " + name + " uses unsupported API version " + std::to_string(major) + "." + std::to_string(minor));
  std::lock_guard<std::mutex> lock(g_mu);
  const std::string key = platform + ":" + name;
  if (Registry().count(key)) return NewError(XLA_FFI_Error_Code_ALREADY_EXISTS, "duplicate FFI handler registration for " + key);
  Registration r;
  r.bundle = a->bundle;
  r.traits = a->traits | metadata.traits;
  r.metadata = metadata;
  Registry()[key] = r;
  return nullptr;
}

XLA_FFI_Error* StreamGet(XLA_FFI_Stream_Get_Args* a) {
  a->stream = a->ctx->stream;
  return nullptr;
}
XLA_FFI_Error* DeviceOrdinalGet(XLA_FFI_DeviceOrdinal_Get_Args* a) {
  a->device_ordinal = a->ctx->device_ordinal;
  return nullptr;
}
XLA_FFI_Error* RunIdGet(XLA_FFI_RunId_Get_Args* a) {
  a->run_id = a->ctx->run_id;
  return nullptr;
}
XLA_FFI_Error* TypeRegister(XLA_FFI_Type_Register_Args* a) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (a->type_id->type_id == 0) a->type_id->type_id = g_next_type_id++;
  return nullptr;
}
XLA_FFI_Error* StateSet(XLA_FFI_State_Set_Args* a) {
  if (a->ctx->state == nullptr) return NewError(XLA_FFI_Error_Code_FAILED_PRECONDITION, "no execution state");
  if (a->ctx->state->count(a->stage)) return NewError(XLA_FFI_Error_Code_ALREADY_EXISTS, "state already set");
  (*a->ctx->state)[a->stage] = {a->type_id->type_id, a->state};
  return nullptr;
}
XLA_FFI_Error* StateGet(XLA_FFI_State_Get_Args* a) {
  if (a->ctx->state == nullptr || !a->ctx->state->count(a->stage))
    return NewError(XLA_FFI_Error_Code_NOT_FOUND, "state not set");
  auto& s = (*a->ctx->state)[a->stage];
  if (s.first != a->type_id->type_id) return NewError(XLA_FFI_Error_Code_INVALID_ARGUMENT, "state type mismatch");
  a->state = s.second;
  return nullptr;
}
// Services the scaled-dot handlers must never need.  Each returns UNIMPLEMENTED so that a test
// notices immediately if a handler starts depending on one of them (in particular on device
// allocation inside `execute`, which a command-buffer compatible handler may not do).
XLA_FFI_Error* InvokeContextGet(XLA_FFI_InvokeContext_Get_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: InvokeContext_Get"); }
XLA_FFI_Error* DeviceMemoryAllocate(XLA_FFI_DeviceMemory_Allocate_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: DeviceMemory_Allocate"); }
XLA_FFI_Error* DeviceMemoryFree(XLA_FFI_DeviceMemory_Free_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: DeviceMemory_Free"); }
XLA_FFI_Error* ThreadPoolSchedule(XLA_FFI_ThreadPool_Schedule_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: ThreadPool_Schedule"); }
XLA_FFI_Error* ThreadPoolNumThreads(XLA_FFI_ThreadPool_NumThreads_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: ThreadPool_NumThreads"); }
XLA_FFI_Error* FutureCreate(XLA_FFI_Future_Create_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: Future_Create"); }
XLA_FFI_Error* FutureSetAvailable(XLA_FFI_Future_SetAvailable_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: Future_SetAvailable"); }
XLA_FFI_Error* FutureSetError(XLA_FFI_Future_SetError_Args*) { return NewError(XLA_FFI_Error_Code_UNIMPLEMENTED, "mock: Future_SetError"); }
XLA_FFI_Error* FindExtension(XLA_FFI_InvokeContext_FindExtension_Args* a) {
  a->extension = nullptr;
  return NewError(XLA_FFI_Error_Code_NOT_FOUND, "mock: no context extensions");
}

const XLA_FFI_Api* Api() {
  static XLA_FFI_Api api = [] {
    XLA_FFI_Api a{};
    a.struct_size = XLA_FFI_Api_STRUCT_SIZE;
    a.api_version.struct_size = XLA_FFI_Api_Version_STRUCT_SIZE;
    a.api_version.major_version = XLA_FFI_API_MAJOR;
    a.api_version.minor_version = XLA_FFI_API_MINOR;
    a.XLA_FFI_Error_Create = ErrorCreate;
    a.XLA_FFI_Error_GetDetails = ErrorGetDetails;
    a.XLA_FFI_Error_Destroy = ErrorDestroy;
    a.XLA_FFI_Handler_Register = HandlerRegister;
    a.XLA_FFI_Stream_Get = StreamGet;
    a.XLA_FFI_Type_Register = TypeRegister;
    a.XLA_FFI_InvokeContext_Get = InvokeContextGet;
    a.XLA_FFI_State_Set = StateSet;
    a.XLA_FFI_State_Get = StateGet;
    a.XLA_FFI_DeviceMemory_Allocate = DeviceMemoryAllocate;
    a.XLA_FFI_DeviceMemory_Free = DeviceMemoryFree;
    a.XLA_FFI_ThreadPool_Schedule = ThreadPoolSchedule;
    a.XLA_FFI_ThreadPool_NumThreads = ThreadPoolNumThreads;
    a.XLA_FFI_Future_Create = FutureCreate;
    a.XLA_FFI_Future_SetAvailable = FutureSetAvailable;
    a.XLA_FFI_Future_SetError = FutureSetError;
    a.XLA_FFI_RunId_Get = RunIdGet;
    a.XLA_FFI_DeviceOrdinal_Get = DeviceOrdinalGet;
    a.XLA_FFI_InvokeContext_FindExtension = FindExtension;
    return a;
  }();
  return &api;
}

// ---- call-frame builder (what xla::ffi::CallFrameBuilder does on the XLA side) --------------
struct Attr {
  std::string name;
  XLA_FFI_AttrType type;
  XLA_FFI_DataType dtype;
  std::vector<uint8_t> bytes;     // scalar value, array payload or string characters
  size_t count = 0;               // array length
};

struct Call {
  std::string target;
  struct Buf {
    XLA_FFI_DataType dtype;
    void* data;
    std::vector<int64_t> dims;
  };
  std::vector<Buf> args, rets;
  std::vector<Attr> attrs;
  std::map<int, std::pair<int64_t, void*>> state;
  bool instantiated = false;
};

struct BuiltFrame {
  std::vector<XLA_FFI_Buffer> arg_bufs, ret_bufs;
  std::vector<XLA_FFI_ArgType> arg_types;
  std::vector<XLA_FFI_RetType> ret_types;
  std::vector<void*> arg_ptrs, ret_ptrs;
  std::vector<Attr> attrs;                      // sorted copy
  std::vector<XLA_FFI_ByteSpan> name_spans, str_spans;
  std::vector<XLA_FFI_ByteSpan*> name_ptrs;
  std::vector<XLA_FFI_Scalar> scalars;
  std::vector<XLA_FFI_Array> arrays;
  std::vector<XLA_FFI_AttrType> attr_types;
  std::vector<void*> attr_ptrs;
  XLA_FFI_CallFrame frame{};
};

void Build(Call& c, bool null_data, XLA_FFI_InvokeContext* ctx, XLA_FFI_ExecutionStage stage, BuiltFrame* b) {
  auto fill = [&](std::vector<Call::Buf>& src, std::vector<XLA_FFI_Buffer>& dst) {
    dst.resize(src.size());
    for (size_t i = 0; i < src.size(); ++i) {
      dst[i] = XLA_FFI_Buffer{};
      dst[i].struct_size = XLA_FFI_Buffer_STRUCT_SIZE;
      dst[i].dtype = src[i].dtype;
      dst[i].data = null_data ? nullptr : src[i].data;
      dst[i].rank = static_cast<int64_t>(src[i].dims.size());
      dst[i].dims = src[i].dims.data();
    }
  };
  fill(c.args, b->arg_bufs);
  fill(c.rets, b->ret_bufs);
  b->arg_types.assign(c.args.size(), XLA_FFI_ArgType_BUFFER);
  b->ret_types.assign(c.rets.size(), XLA_FFI_RetType_BUFFER);
  for (auto& x : b->arg_bufs) b->arg_ptrs.push_back(&x);
  for (auto& x : b->ret_bufs) b->ret_ptrs.push_back(&x);

  b->attrs = c.attrs;   // attributes are handed over sorted by name (c_api.h:478-480)
  std::sort(b->attrs.begin(), b->attrs.end(), [](const Attr& x, const Attr& y) { return x.name < y.name; });
  const size_t n = b->attrs.size();
  b->name_spans.resize(n);
  b->str_spans.resize(n);
  b->scalars.resize(n);
  b->arrays.resize(n);
  for (size_t i = 0; i < n; ++i) {
    Attr& at = b->attrs[i];
    b->name_spans[i] = XLA_FFI_ByteSpan{at.name.data(), at.name.size()};
    b->attr_types.push_back(at.type);
    switch (at.type) {
      case XLA_FFI_AttrType_SCALAR:
        b->scalars[i] = XLA_FFI_Scalar{at.dtype, at.bytes.data()};
        b->attr_ptrs.push_back(&b->scalars[i]);
        break;
      case XLA_FFI_AttrType_ARRAY:
        b->arrays[i] = XLA_FFI_Array{at.dtype, at.count, at.bytes.data()};
        b->attr_ptrs.push_back(&b->arrays[i]);
        break;
      default:
        b->str_spans[i] = XLA_FFI_ByteSpan{reinterpret_cast<const char*>(at.bytes.data()), at.bytes.size()};
        b->attr_ptrs.push_back(&b->str_spans[i]);
        break;
    }
  }
  for (auto& s : b->name_spans) b->name_ptrs.push_back(&s);

  XLA_FFI_CallFrame& f = b->frame;
  f.struct_size = XLA_FFI_CallFrame_STRUCT_SIZE;
  f.api = Api();
  f.ctx = ctx;
  f.stage = stage;
  f.args.struct_size = XLA_FFI_Args_STRUCT_SIZE;
  f.args.size = static_cast<int64_t>(c.args.size());
  f.args.types = b->arg_types.data();
  f.args.args = b->arg_ptrs.data();
  f.rets.struct_size = XLA_FFI_Rets_STRUCT_SIZE;
  f.rets.size = static_cast<int64_t>(c.rets.size());
  f.rets.types = b->ret_types.data();
  f.rets.rets = b->ret_ptrs.data();
  f.attrs.struct_size = XLA_FFI_Attrs_STRUCT_SIZE;
  f.attrs.size = static_cast<int64_t>(n);
  f.attrs.types = b->attr_types.data();
  f.attrs.names = b->name_ptrs.data();
  f.attrs.attrs = b->attr_ptrs.data();
}

int Finish(XLA_FFI_Error* e, char* err, size_t err_len) {
  if (e == nullptr) {
    if (err && err_len) err[0] = '\0';
    return 0;
  }
  if (err && err_len) snprintf(err, err_len, "%s", e->message.c_str());
  const int code = static_cast<int>(e->code);
  delete e;
  return code ? code : static_cast<int>(XLA_FFI_Error_Code_UNKNOWN);
}

XLA_FFI_Handler* StageHandler(const Registration& r, int stage) {
  switch (stage) {
    case XLA_FFI_ExecutionStage_INSTANTIATE: return r.bundle.instantiate;
    case XLA_FFI_ExecutionStage_PREPARE: return r.bundle.prepare;
    case XLA_FFI_ExecutionStage_INITIALIZE: return r.bundle.initialize;
    case XLA_FFI_ExecutionStage_EXECUTE: return r.bundle.execute;
    default: return nullptr;
  }
}

void AddScalar(Call* c, const char* name, XLA_FFI_DataType dtype, const void* value, size_t size) {
  Attr a;
  a.name = name;
  a.type = XLA_FFI_AttrType_SCALAR;
  a.dtype = dtype;
  a.bytes.assign(static_cast<const uint8_t*>(value), static_cast<const uint8_t*>(value) + size);
  c->attrs.push_back(std::move(a));
}

}  // namespace

MOCK_EXPORT const void* mockffi_api() { return Api(); }

// dlopen()s a handler library and calls its `int <register_symbol>(const XLA_FFI_Api*, char*, size_t)`.
MOCK_EXPORT int mockffi_load_library(const char* path, const char* register_symbol, char* err, size_t err_len) {
  void* lib = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  if (lib == nullptr) {
    if (err && err_len) snprintf(err, err_len, "dlopen(%s): %s", path, dlerror());
    return XLA_FFI_Error_Code_NOT_FOUND;
  }
  using RegisterFn = int (*)(const void*, char*, size_t);
  auto fn = reinterpret_cast<RegisterFn>(dlsym(lib, register_symbol));
  if (fn == nullptr) {
    if (err && err_len) snprintf(err, err_len, "dlsym(%s): not found", register_symbol);
    return XLA_FFI_Error_Code_NOT_FOUND;
  }
  return fn(Api(), err, err_len);
}

// 1 when `platform:target` is registered; traits (if not null) receives the handler traits.
MOCK_EXPORT int mockffi_find_handler(const char* target, const char* platform, uint32_t* traits, int* api_minor) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = Registry().find(std::string(platform) + ":" + target);
  if (it == Registry().end()) return 0;
  if (traits) *traits = it->second.traits;
  if (api_minor) *api_minor = it->second.metadata.api_version.minor_version;
  return 1;
}

MOCK_EXPORT void* mockffi_call_new(const char* target) {
  auto* c = new Call();
  c->target = target;
  return c;
}
MOCK_EXPORT void mockffi_call_free(void* call) { delete static_cast<Call*>(call); }
MOCK_EXPORT void mockffi_call_add_arg(void* call, int dtype, void* data, int rank, const int64_t* dims) {
  static_cast<Call*>(call)->args.push_back({static_cast<XLA_FFI_DataType>(dtype), data, std::vector<int64_t>(dims, dims + rank)});
}
MOCK_EXPORT void mockffi_call_add_ret(void* call, int dtype, void* data, int rank, const int64_t* dims) {
  static_cast<Call*>(call)->rets.push_back({static_cast<XLA_FFI_DataType>(dtype), data, std::vector<int64_t>(dims, dims + rank)});
}
// Re-points an operand / result at a new device address (XLA's UpdateWithBuffers).
MOCK_EXPORT void mockffi_call_set_arg_data(void* call, int index, void* data) { static_cast<Call*>(call)->args.at(index).data = data; }
MOCK_EXPORT void mockffi_call_set_ret_data(void* call, int index, void* data) { static_cast<Call*>(call)->rets.at(index).data = data; }
MOCK_EXPORT void mockffi_call_attr_i64(void* call, const char* name, int64_t v) { AddScalar(static_cast<Call*>(call), name, XLA_FFI_DataType_S64, &v, sizeof(v)); }
MOCK_EXPORT void mockffi_call_attr_i32(void* call, const char* name, int32_t v) { AddScalar(static_cast<Call*>(call), name, XLA_FFI_DataType_S32, &v, sizeof(v)); }
MOCK_EXPORT void mockffi_call_attr_f64(void* call, const char* name, double v) { AddScalar(static_cast<Call*>(call), name, XLA_FFI_DataType_F64, &v, sizeof(v)); }
MOCK_EXPORT void mockffi_call_attr_f32(void* call, const char* name, float v) { AddScalar(static_cast<Call*>(call), name, XLA_FFI_DataType_F32, &v, sizeof(v)); }
MOCK_EXPORT void mockffi_call_attr_bool(void* call, const char* name, int v) {
  const uint8_t b = v ? 1 : 0;
  AddScalar(static_cast<Call*>(call), name, XLA_FFI_DataType_PRED, &b, sizeof(b));
}
MOCK_EXPORT void mockffi_call_attr_str(void* call, const char* name, const char* v) {
  Attr a;
  a.name = name;
  a.type = XLA_FFI_AttrType_STRING;
  a.dtype = XLA_FFI_DataType_INVALID;
  a.bytes.assign(reinterpret_cast<const uint8_t*>(v), reinterpret_cast<const uint8_t*>(v) + strlen(v));
  static_cast<Call*>(call)->attrs.push_back(std::move(a));
}
MOCK_EXPORT void mockffi_call_attr_i64_array(void* call, const char* name, const int64_t* v, size_t count) {
  Attr a;
  a.name = name;
  a.type = XLA_FFI_AttrType_ARRAY;
  a.dtype = XLA_FFI_DataType_S64;
  a.count = count;
  a.bytes.assign(reinterpret_cast<const uint8_t*>(v), reinterpret_cast<const uint8_t*>(v + count));
  static_cast<Call*>(call)->attrs.push_back(std::move(a));
}

// Runs one stage of the call.  INSTANTIATE hides the buffer addresses, as XLA does.
MOCK_EXPORT int mockffi_call_invoke(void* call, int stage, void* stream, int device_ordinal, char* err, size_t err_len) {
  Call* c = static_cast<Call*>(call);
  Registration reg;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = Registry().find("CUDA:" + c->target);
    if (it == Registry().end()) {
      if (err && err_len) snprintf(err, err_len, "No FFI handler registered for %s on platform CUDA", c->target.c_str());
      return XLA_FFI_Error_Code_NOT_FOUND;
    }
    reg = it->second;
  }
  XLA_FFI_Handler* h = StageHandler(reg, stage);
  if (h == nullptr) {   // optional stage not provided: nothing to do
    if (err && err_len) err[0] = '\0';
    return 0;
  }
  XLA_FFI_InvokeContext ctx;
  ctx.stream = stage >= XLA_FFI_ExecutionStage_INITIALIZE ? stream : nullptr;
  ctx.device_ordinal = device_ordinal;
  ctx.state = &c->state;
  BuiltFrame built;
  Build(*c, stage == XLA_FFI_ExecutionStage_INSTANTIATE, &ctx, static_cast<XLA_FFI_ExecutionStage>(stage), &built);
  return Finish(h(&built.frame), err, err_len);
}

// The whole life of a call site: instantiate (first time only) -> prepare -> initialize -> execute.
MOCK_EXPORT int mockffi_call_run(void* call, void* stream, int device_ordinal, char* err, size_t err_len) {
  Call* c = static_cast<Call*>(call);
  if (!c->instantiated) {
    if (int rc = mockffi_call_invoke(call, XLA_FFI_ExecutionStage_INSTANTIATE, nullptr, device_ordinal, err, err_len)) return rc;
    c->instantiated = true;
  }
  for (int stage : {XLA_FFI_ExecutionStage_PREPARE, XLA_FFI_ExecutionStage_INITIALIZE, XLA_FFI_ExecutionStage_EXECUTE}) {
    if (int rc = mockffi_call_invoke(call, stage, stream, device_ordinal, err, err_len)) return rc;
  }
  return 0;
}

// Execute stage only (the steady state of a compiled executable).
MOCK_EXPORT int mockffi_call_execute(void* call, void* stream, int device_ordinal, char* err, size_t err_len) {
  return mockffi_call_invoke(call, XLA_FFI_ExecutionStage_EXECUTE, stream, device_ordinal, err, err_len);
}
