// Worker messages in native form.
//
// The controller's messages reach the worker as pickled tuples whose first element names the
// kind.  The kinds that the native core executes itself are decoded into the structs below
// on arrival (WorkerCore::route_batch, define_recording) and never touch Python again:
// operator calls, shape-only calls of null-device workers, deletions, and the items of a
// recording.  The remaining kinds (collectives, borrows, sends, pipes, actor calls, process
// groups) are dispatched by name to the worker actor's Python methods.
//
// Parity: monarch_messages/src/worker.rs (WorkerMessage: CallFunction, DeleteRefs,
// DefineRecording / CallRecording, ...; CallFunctionError with its dependent form).
#pragma once

#include <torch/extension.h>

#include <ATen/core/dispatch/Dispatcher.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <variant>
#include <vector>

namespace mb::tensor {

namespace py = pybind11;

enum class MessageKind {
  Call,            // ("call", seq, results, mutates, fspec, args, kwargs, stream[, metas])
  Delete,          // ("delete", ids)
  CreateStream,
  BorrowCreate,
  BorrowDrop,
  Reduce,
  SendTensor,
  DefineRecording,
  CallRecording,
  Other,           // everything the Python router names by itself
};

inline MessageKind kind_of(const char* name) {
  if (name == nullptr) return MessageKind::Other;
  if (std::strcmp(name, "call") == 0) return MessageKind::Call;
  if (std::strcmp(name, "delete") == 0) return MessageKind::Delete;
  if (std::strcmp(name, "create_stream") == 0) return MessageKind::CreateStream;
  if (std::strcmp(name, "borrow_create") == 0) return MessageKind::BorrowCreate;
  if (std::strcmp(name, "borrow_drop") == 0) return MessageKind::BorrowDrop;
  if (std::strcmp(name, "reduce") == 0) return MessageKind::Reduce;
  if (std::strcmp(name, "send_tensor") == 0) return MessageKind::SendTensor;
  if (std::strcmp(name, "define_recording") == 0) return MessageKind::DefineRecording;
  if (std::strcmp(name, "call_recording") == 0) return MessageKind::CallRecording;
  return MessageKind::Other;
}

// A failed invocation as the worker remembers it (CallFunctionError): results of a failed
// call hold one of these, and calls that read them inherit it with dependent_of set.
struct RemoteErr {
  int64_t seq, rank;
  std::string func, text, tb;
  int64_t dependent_of;  // -1: original failure
};
using ErrPtr = std::shared_ptr<RemoteErr>;
using Value = std::variant<std::monostate, at::Tensor, ErrPtr, py::object>;

struct Arg {           // one positional or keyword argument of a recorded call
  enum Kind { Const, RefOne, RefList } kind = Const;
  c10::IValue constant;
  std::vector<int64_t> refs;
  std::string name;    // keyword name ("" = positional)
};

// CallFunction for an ATen operator, resolved against the dispatcher.
struct OpCall {
  int64_t seq = 0;
  std::vector<int64_t> results, mutates;
  std::string name;
  c10::OperatorHandle op;
  std::vector<Arg> args;
  int64_t stream = 0;
  // torch.cuda.Stream to enter around the launch (borrowed: the core's stream table owns
  // it), or null when the executing thread's current stream is already the right one
  PyObject* py_stream = nullptr;
  explicit OpCall(c10::OperatorHandle h) : op(std::move(h)) {}
};

// DeleteRefs.
struct DeleteRefs {
  std::vector<int64_t> ids;
};

// CallFunction on a null-device worker: nothing runs, zero tensors of the announced shapes
// and dtypes stand in for the results.
struct ShapeOnlyCall {
  int64_t seq = 0;
  std::vector<int64_t> results;
  struct Meta {
    std::vector<int64_t> shape;
    at::ScalarType dtype;
  };
  std::vector<Meta> metas;
  int64_t stream = 0;
};

// One item of a recording (DefineRecording).
struct RecItem {
  std::unique_ptr<OpCall> call;  // null: not an operator call -> Python fallback
  size_t index = 0;
  std::vector<int64_t> drop;     // refs of the recording that are dead after this item
};

}  // namespace mb::tensor
