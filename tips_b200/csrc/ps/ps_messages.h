// Wire messages of the host parameter server and the dtype glue.
//
// Field parity with the reference's FlatBuffers schema
// (tips/core/message/ps_messages.fbs:3-43): MessageMeta{client_id, message_id},
// PullRequest{meta, keys[u64], dtypes[], lengths[u32]}, KeyItem{key, dtype,
// value[u8]}, PullResponse{meta, data[KeyItem]}, PushRequest{meta,
// data[KeyItem]}, PushResponse{meta}; and with tips/core/ps/ps_utils.cc:7-37
// (ToDatatype / ToMessageDataType), which is the identity here because the wire
// uses the runtime's own Datatype codes.  Encoded with NaiveBuffer.
#pragma once

#include <cstring>
#include <string>
#include <vector>

#include "core/datatype.h"
#include "core/naive_buffer.h"

namespace tips {
namespace ps {

struct MessageMeta {
  int32_t client_id{0};
  uint64_t message_id{0};
};

struct KeyItem {
  uint64_t key{0};
  Datatype dtype{Datatype::kFp32};
  std::vector<uint8_t> value;  // raw little-endian elements
};

struct PullRequest {
  MessageMeta meta;
  std::vector<uint64_t> keys;
  std::vector<int32_t> dtypes;
  std::vector<uint32_t> lengths;
  void Serialize(NaiveBuffer* b) const { *b << meta.client_id << meta.message_id << keys << dtypes << lengths; }
  void Deserialize(NaiveBuffer* b) { *b >> meta.client_id >> meta.message_id >> keys >> dtypes >> lengths; }
};

inline void SerializeItems(NaiveBuffer* b, const std::vector<KeyItem>& items) {
  *b << static_cast<uint64_t>(items.size());
  for (const KeyItem& it : items) *b << it.key << static_cast<int32_t>(it.dtype) << it.value;
}
inline void DeserializeItems(NaiveBuffer* b, std::vector<KeyItem>* items) {
  uint64_t n = 0;
  *b >> n;
  items->resize(n);
  for (KeyItem& it : *items) {
    int32_t dt = 0;
    *b >> it.key >> dt >> it.value;
    it.dtype = static_cast<Datatype>(dt);
  }
}

struct PullResponse {
  MessageMeta meta;
  std::vector<KeyItem> data;  // in request order
  void Serialize(NaiveBuffer* b) const {
    *b << meta.client_id << meta.message_id;
    SerializeItems(b, data);
  }
  void Deserialize(NaiveBuffer* b) {
    *b >> meta.client_id >> meta.message_id;
    DeserializeItems(b, &data);
  }
};

struct PushRequest {
  MessageMeta meta;
  std::vector<KeyItem> data;
  void Serialize(NaiveBuffer* b) const {
    *b << meta.client_id << meta.message_id;
    SerializeItems(b, data);
  }
  void Deserialize(NaiveBuffer* b) {
    *b >> meta.client_id >> meta.message_id;
    DeserializeItems(b, &data);
  }
};

struct PushResponse {
  MessageMeta meta;
  void Serialize(NaiveBuffer* b) const { *b << meta.client_id << meta.message_id; }
  void Deserialize(NaiveBuffer* b) { *b >> meta.client_id >> meta.message_id; }
};

// Uniform requests (every row of one dtype and one length, which is what an embedding table sends) travel packed:
// the keys as one array and the rows as one block, instead of one KeyItem with its own byte vector per row.
//   packed pull request   meta, dtype, length, keys[u64]
//   packed pull response  meta, n, bad, then n * length elements (request order; `bad` = rows that exist on the
//                         server with another dtype or length: their slots are zero)
//   packed push request   meta, dtype, length, keys[u64], then keys.size() * length elements
//   packed push response  PushResponse followed by the number of rows that did not exist
struct PackedHeader {
  MessageMeta meta;
  Datatype dtype{Datatype::kFp32};
  uint32_t length{0};
  std::vector<uint64_t> keys;
  void Serialize(NaiveBuffer* b) const {
    *b << meta.client_id << meta.message_id << static_cast<int32_t>(dtype) << length << keys;
  }
  void Deserialize(NaiveBuffer* b) {
    int32_t dt = 0;
    *b >> meta.client_id >> meta.message_id >> dt >> length >> keys;
    dtype = static_cast<Datatype>(dt);
  }
  size_t row_bytes() const { return DatatypeNumBytes(dtype) * length; }
  // Bytes this header takes at the start of a message of `size` bytes (0: the message is too short), so that a
  // reader can parse the header alone and leave the row block where it is.
  static size_t EncodedSize(const void* message, size_t size) {
    constexpr size_t fixed = sizeof(int32_t) + sizeof(uint64_t) + sizeof(int32_t) + sizeof(uint32_t);
    if (size < fixed + sizeof(uint64_t)) return 0;
    uint64_t n = 0;
    memcpy(&n, static_cast<const char*>(message) + fixed, sizeof(n));
    const size_t total = fixed + sizeof(uint64_t) + n * sizeof(uint64_t);
    return n <= size && total <= size ? total : 0;
  }
};

inline Datatype ToDatatype(int32_t message_dtype) { return static_cast<Datatype>(message_dtype); }
inline int32_t ToMessageDataType(Datatype t) { return static_cast<int32_t>(t); }

// Names of the RPC services (reference: tips/core/rpc_service_names.h:8-9).
constexpr const char* kPullServiceName = "pull_service";
constexpr const char* kPushServiceName = "push_service";
constexpr const char* kPackedPullServiceName = "pull_packed_service";
constexpr const char* kPackedPushServiceName = "push_packed_service";

}  // namespace ps
}  // namespace tips
