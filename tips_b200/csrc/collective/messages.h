// Negotiation messages of the collective engine.
//
// Field parity with the reference's FlatBuffers schema
// (tips/core/message/collective_messages.fbs:3-38): RequestMessage{request_rank,
// request_type, tensor_type, tensor_name, tensor_shape}; ResponseMessage{
// response_type (ERROR=-2, SHUTDOWN=-1, ALLREDUCE, ALLGATHER, BROADCAST),
// tensor_name, error_message, tensor_sizes}.  Added fields carry what the
// reference hard-wires or drops: the broadcast root, the reduction operator,
// pre/post scale factors and the device kind, so they can be validated across
// ranks; a response may name several tensors that are executed as one fused
// group.  Encoding is the NaiveBuffer wire format (FlatBuffers is not on the
// target image).
#pragma once

#include <string>
#include <vector>

#include "core/datatype.h"
#include "core/naive_buffer.h"

namespace tips {
namespace collective {

enum class RequestType : int16_t { kAllreduce = 0, kAllgather = 1, kBroadcast = 2 };
enum class ResponseType : int16_t { kError = -2, kShutdown = -1, kAllreduce = 0, kAllgather = 1, kBroadcast = 2 };

const char* RequestTypeName(RequestType t);

struct RequestMessage {
  int32_t request_rank{0};
  RequestType request_type{RequestType::kAllreduce};
  Datatype tensor_type{Datatype::kFp32};
  std::string tensor_name;
  std::vector<int64_t> tensor_shape;
  int32_t root_rank{0};
  int32_t reduce_op{0};
  int32_t device{0};  // 0 = host memory, 1 = CUDA device memory
  double prescale{1.0};
  double postscale{1.0};

  void Serialize(NaiveBuffer* buf) const;
  void Deserialize(NaiveBuffer* buf);
  int64_t NumElements() const;
};

struct ResponseMessage {
  ResponseType response_type{ResponseType::kError};
  // One or more tensors executed together; all share type, dtype and operator.
  std::vector<std::string> tensor_names;
  std::string error_message;
  // Allgather: first-dimension size contributed by every rank.
  std::vector<int64_t> tensor_sizes;
  int32_t root_rank{0};

  void Serialize(NaiveBuffer* buf) const;
  void Deserialize(NaiveBuffer* buf);
};

}  // namespace collective
}  // namespace tips
