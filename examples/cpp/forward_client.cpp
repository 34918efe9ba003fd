// /forward client in plain C++ (POSIX sockets, no third-party library): packs one request as msgpack, posts it,
// unpacks the answer and prints every returned tensor.
//
//   g++ -O2 -std=c++17 -o forward_client examples/cpp/forward_client.cpp
//   ./forward_client 127.0.0.1 8080 1 2 3 4 5
//
// Request schema (the same one the reference documents in src/ksana_llm/cpp/README.md and exercises in
// src/ksana_llm/cpp/serving_forward_client.cpp):
//   {"requests": [{"input_tokens": [...], "request_target": [
//       {"target_name": "transformer" | "layernorm" | "logits" | "lm_head",
//        "slice_pos": [[first, last], ...] or "token_id": [...],
//        "token_reduce_mode": "GATHER_ALL" | "GATHER_TOKEN_ID", "cutoff_layer": n (lm_head only)}]}]}
// Answer: {"responses": [{"input_token_ids": [...], "response": [
//       {"target_name": ..., "tensor": {"data": base64 of float32 values, "shape": [...], "dtype": "float32"}}]}]}
#include <arpa/inet.h>
#include <netdb.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

// ---- msgpack writer (the subset a request needs) ----------------------------------------------------------
struct Packer {
  std::string out;
  void Byte(uint8_t b) { out.push_back(static_cast<char>(b)); }
  void Be(uint64_t v, int bytes) {
    for (int i = bytes - 1; i >= 0; --i) Byte(static_cast<uint8_t>(v >> (8 * i)));
  }
  void Map(uint32_t n) {
    if (n < 16) Byte(0x80 | n); else { Byte(0xde); Be(n, 2); }
  }
  void Array(uint32_t n) {
    if (n < 16) Byte(0x90 | n); else if (n < 65536) { Byte(0xdc); Be(n, 2); } else { Byte(0xdd); Be(n, 4); }
  }
  void Str(const std::string& s) {
    if (s.size() < 32) Byte(0xa0 | s.size()); else if (s.size() < 256) { Byte(0xd9); Be(s.size(), 1); }
    else { Byte(0xda); Be(s.size(), 2); }
    out += s;
  }
  void Int(int64_t v) {
    if (v >= 0 && v < 128) Byte(static_cast<uint8_t>(v));
    else if (v < 0 && v >= -32) Byte(static_cast<uint8_t>(v));
    else { Byte(0xd3); Be(static_cast<uint64_t>(v), 8); }
  }
};

// ---- msgpack reader (generic value tree) ------------------------------------------------------------------
struct Value {
  enum Kind { kNil, kBool, kInt, kFloat, kStr, kArray, kMap } kind = kNil;
  int64_t i = 0;
  double f = 0;
  std::string s;  // str and bin
  std::vector<Value> items;
  std::vector<std::pair<Value, Value>> fields;
  const Value& At(const std::string& key) const {
    for (const auto& kv : fields)
      if (kv.first.kind == kStr && kv.first.s == key) return kv.second;
    throw std::runtime_error("missing key " + key);
  }
};

struct Unpacker {
  const uint8_t* p;
  const uint8_t* end;
  uint64_t Be(int bytes) {
    if (end - p < bytes) throw std::runtime_error("truncated msgpack");
    uint64_t v = 0;
    for (int k = 0; k < bytes; ++k) v = (v << 8) | *p++;
    return v;
  }
  Value Bytes(size_t n) {
    if (static_cast<size_t>(end - p) < n) throw std::runtime_error("truncated msgpack");
    Value v;
    v.kind = Value::kStr;
    v.s.assign(reinterpret_cast<const char*>(p), n);
    p += n;
    return v;
  }
  Value Seq(size_t n, bool map) {
    Value v;
    v.kind = map ? Value::kMap : Value::kArray;
    for (size_t k = 0; k < n; ++k) {
      if (map) { Value key = Next(); v.fields.emplace_back(std::move(key), Next()); }
      else v.items.push_back(Next());
    }
    return v;
  }
  Value Next() {
    uint8_t t = static_cast<uint8_t>(Be(1));
    Value v;
    if (t < 0x80) { v.kind = Value::kInt; v.i = t; return v; }
    if (t >= 0xe0) { v.kind = Value::kInt; v.i = static_cast<int8_t>(t); return v; }
    if ((t & 0xf0) == 0x80) return Seq(t & 0x0f, true);
    if ((t & 0xf0) == 0x90) return Seq(t & 0x0f, false);
    if ((t & 0xe0) == 0xa0) return Bytes(t & 0x1f);
    switch (t) {
      case 0xc0: return v;
      case 0xc2: case 0xc3: v.kind = Value::kBool; v.i = t == 0xc3; return v;
      case 0xc4: case 0xd9: return Bytes(Be(1));
      case 0xc5: case 0xda: return Bytes(Be(2));
      case 0xc6: case 0xdb: return Bytes(Be(4));
      case 0xca: { uint32_t b = static_cast<uint32_t>(Be(4)); float x; std::memcpy(&x, &b, 4);
                   v.kind = Value::kFloat; v.f = x; return v; }
      case 0xcb: { uint64_t b = Be(8); std::memcpy(&v.f, &b, 8); v.kind = Value::kFloat; return v; }
      case 0xcc: v.kind = Value::kInt; v.i = Be(1); return v;
      case 0xcd: v.kind = Value::kInt; v.i = Be(2); return v;
      case 0xce: v.kind = Value::kInt; v.i = Be(4); return v;
      case 0xcf: v.kind = Value::kInt; v.i = static_cast<int64_t>(Be(8)); return v;
      case 0xd0: v.kind = Value::kInt; v.i = static_cast<int8_t>(Be(1)); return v;
      case 0xd1: v.kind = Value::kInt; v.i = static_cast<int16_t>(Be(2)); return v;
      case 0xd2: v.kind = Value::kInt; v.i = static_cast<int32_t>(Be(4)); return v;
      case 0xd3: v.kind = Value::kInt; v.i = static_cast<int64_t>(Be(8)); return v;
      case 0xdc: return Seq(Be(2), false);
      case 0xdd: return Seq(Be(4), false);
      case 0xde: return Seq(Be(2), true);
      case 0xdf: return Seq(Be(4), true);
      default: throw std::runtime_error("unsupported msgpack type");
    }
  }
};

std::string Base64Decode(const std::string& in) {
  std::string out;
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : in) {
    int v;
    if (c >= 'A' && c <= 'Z') v = c - 'A';
    else if (c >= 'a' && c <= 'z') v = c - 'a' + 26;
    else if (c >= '0' && c <= '9') v = c - '0' + 52;
    else if (c == '+') v = 62;
    else if (c == '/') v = 63;
    else continue;  // '=' and line breaks
    acc = (acc << 6) | static_cast<uint32_t>(v);
    bits += 6;
    if (bits >= 8) { bits -= 8; out.push_back(static_cast<char>((acc >> bits) & 0xff)); }
  }
  return out;
}

// ---- HTTP POST over a TCP socket --------------------------------------------------------------------------
std::string Post(const std::string& host, const std::string& port, const std::string& path, const std::string& body) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || res == nullptr)
    throw std::runtime_error("cannot resolve " + host);
  int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
  if (fd < 0 || connect(fd, res->ai_addr, res->ai_addrlen) != 0) {
    freeaddrinfo(res);
    throw std::runtime_error("cannot connect to " + host + ":" + port);
  }
  freeaddrinfo(res);
  std::string req = "POST " + path + " HTTP/1.1\r\nHost: " + host + ":" + port +
                    "\r\nContent-Type: application/x-msgpack\r\nConnection: close\r\nContent-Length: " +
                    std::to_string(body.size()) + "\r\n\r\n" + body;
  for (size_t sent = 0; sent < req.size();) {
    ssize_t n = send(fd, req.data() + sent, req.size() - sent, 0);
    if (n <= 0) { close(fd); throw std::runtime_error("send failed"); }
    sent += static_cast<size_t>(n);
  }
  std::string resp;
  char buf[65536];
  for (ssize_t n; (n = recv(fd, buf, sizeof buf, 0)) > 0;) resp.append(buf, static_cast<size_t>(n));
  close(fd);
  size_t head = resp.find("\r\n\r\n");
  if (head == std::string::npos) throw std::runtime_error("malformed HTTP answer");
  if (resp.compare(0, 12, "HTTP/1.1 200") != 0) throw std::runtime_error("server answered: " + resp.substr(0, resp.find("\r\n")));
  std::string headers = resp.substr(0, head), payload = resp.substr(head + 4);
  for (auto& c : headers) c = static_cast<char>(tolower(c));
  if (headers.find("transfer-encoding: chunked") != std::string::npos) {  // size line, data, CRLF, ... 0
    std::string joined;
    for (size_t at = 0; at < payload.size();) {
      size_t eol = payload.find("\r\n", at);
      if (eol == std::string::npos) break;
      size_t n = std::strtoul(payload.substr(at, eol - at).c_str(), nullptr, 16);
      if (n == 0) break;
      joined += payload.substr(eol + 2, n);
      at = eol + 2 + n + 2;
    }
    return joined;
  }
  return payload;
}

}  // namespace

int main(int argc, char** argv) {
  std::string host = argc > 1 ? argv[1] : "127.0.0.1", port = argc > 2 ? argv[2] : "8080";
  std::vector<int64_t> tokens;
  for (int k = 3; k < argc; ++k) tokens.push_back(std::atoll(argv[k]));
  if (tokens.empty()) tokens = {1, 2, 3, 4, 5};
  Packer pk;
  pk.Map(1); pk.Str("requests"); pk.Array(1);
  pk.Map(2);
  pk.Str("input_tokens"); pk.Array(static_cast<uint32_t>(tokens.size()));
  for (int64_t t : tokens) pk.Int(t);
  pk.Str("request_target"); pk.Array(2);
  pk.Map(3);  // the last row after the final norm
  pk.Str("target_name"); pk.Str("layernorm");
  pk.Str("slice_pos"); pk.Array(1); pk.Array(2); pk.Int(-1); pk.Int(-1);
  pk.Str("token_reduce_mode"); pk.Str("GATHER_ALL");
  pk.Map(3);  // probability of every following input token
  pk.Str("target_name"); pk.Str("logits");
  pk.Str("slice_pos"); pk.Array(1); pk.Array(2); pk.Int(0); pk.Int(-2);
  pk.Str("token_reduce_mode"); pk.Str("GATHER_TOKEN_ID");
  try {
    std::string raw = Post(host, port, "/forward", pk.out);
    Unpacker up{reinterpret_cast<const uint8_t*>(raw.data()), reinterpret_cast<const uint8_t*>(raw.data()) + raw.size()};
    Value root = up.Next();
    for (const Value& resp : root.At("responses").items) {
      for (const Value& t : resp.At("response").items) {
        const Value& tensor = t.At("tensor");
        std::string bytes = Base64Decode(tensor.At("data").s);
        std::printf("%s shape=[", t.At("target_name").s.c_str());
        size_t count = 1;
        const auto& shape = tensor.At("shape").items;
        for (size_t d = 0; d < shape.size(); ++d) {
          std::printf(d ? ", %lld" : "%lld", static_cast<long long>(shape[d].i));
          count *= static_cast<size_t>(shape[d].i);
        }
        std::printf("] values=");
        if (bytes.size() != count * sizeof(float)) throw std::runtime_error("tensor size does not match its shape");
        for (size_t k = 0; k < count && k < 8; ++k) {
          float x;
          std::memcpy(&x, bytes.data() + 4 * k, 4);
          std::printf("%s%.6g", k ? " " : "", x);
        }
        std::printf("\n");
      }
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "forward_client: %s\n", e.what());
    return 1;
  }
  return 0;
}
