#include "collective/messages.h"

namespace tips {
namespace collective {

const char* RequestTypeName(RequestType t) {
  switch (t) {
    case RequestType::kAllreduce: return "ALLREDUCE";
    case RequestType::kAllgather: return "ALLGATHER";
    case RequestType::kBroadcast: return "BROADCAST";
  }
  return "?";
}

void RequestMessage::Serialize(NaiveBuffer* buf) const {
  *buf << request_rank << static_cast<int16_t>(request_type) << static_cast<int32_t>(tensor_type) << tensor_name
       << tensor_shape << root_rank << reduce_op << device << prescale << postscale;
}

void RequestMessage::Deserialize(NaiveBuffer* buf) {
  int16_t rt = 0;
  int32_t dt = 0;
  *buf >> request_rank >> rt >> dt >> tensor_name >> tensor_shape >> root_rank >> reduce_op >> device >> prescale >>
      postscale;
  request_type = static_cast<RequestType>(rt);
  tensor_type  = static_cast<Datatype>(dt);
}

int64_t RequestMessage::NumElements() const {
  int64_t n = 1;
  for (int64_t d : tensor_shape) n *= d;
  return n;
}

void ResponseMessage::Serialize(NaiveBuffer* buf) const {
  *buf << static_cast<int16_t>(response_type) << static_cast<uint64_t>(tensor_names.size());
  for (auto& n : tensor_names) *buf << n;
  *buf << error_message << tensor_sizes << root_rank;
}

void ResponseMessage::Deserialize(NaiveBuffer* buf) {
  int16_t rt = 0;
  uint64_t n = 0;
  *buf >> rt >> n;
  response_type = static_cast<ResponseType>(rt);
  tensor_names.resize(n);
  for (auto& s : tensor_names) *buf >> s;
  *buf >> error_message >> tensor_sizes >> root_rank;
}

}  // namespace collective
}  // namespace tips
