#include "actor/reference.h"

namespace mb {

// "world[rank]"
ProcId ProcId::parse(const std::string& s) {
  auto lb = s.rfind('[');
  if (lb == std::string::npos || s.back() != ']') throw CodecError("bad proc id: " + s);
  ProcId p;
  p.world = s.substr(0, lb);
  p.rank = std::stoll(s.substr(lb + 1, s.size() - lb - 2));
  return p;
}

// "world[rank].name[pid]"
ActorId ActorId::parse(const std::string& s) {
  // the actor name follows the first "]." after the proc id
  auto sep = s.find("].");
  if (sep == std::string::npos) throw CodecError("bad actor id: " + s);
  ActorId a;
  a.proc = ProcId::parse(s.substr(0, sep + 1));
  std::string rest = s.substr(sep + 2);
  auto lb = rest.rfind('[');
  if (lb == std::string::npos || rest.back() != ']') throw CodecError("bad actor id: " + s);
  a.name = rest.substr(0, lb);
  a.pid = std::stoll(rest.substr(lb + 1, rest.size() - lb - 2));
  return a;
}

// "world[rank].name[pid][port]"
PortId PortId::parse(const std::string& s) {
  auto lb = s.rfind('[');
  if (lb == std::string::npos || s.back() != ']') throw CodecError("bad port id: " + s);
  PortId p;
  p.actor = ActorId::parse(s.substr(0, lb));
  p.port = std::stoull(s.substr(lb + 1, s.size() - lb - 2));
  return p;
}

std::string Envelope::encode_head() const {
  Writer w;
  write_actor(w, sender);
  write_port(w, dest);
  w.u32((uint32_t)headers.size());
  for (auto& kv : headers) {
    w.str(kv.first);
    w.str(kv.second);
  }
  w.u64(data.size());
  w.u32((uint32_t)parts.size());
  for (auto& p : parts) w.u64(p.size());
  return std::move(w.buf);
}

std::string Envelope::encode() const {
  std::string out = encode_head();
  out.append(data);
  for (auto& p : parts) out.append(p);
  return out;
}

Envelope Envelope::decode(std::string_view bytes) {
  Reader r(bytes);
  Envelope e;
  e.sender = read_actor(r);
  e.dest = read_port(r);
  uint32_t nh = r.u32();
  for (uint32_t i = 0; i < nh; ++i) {
    std::string k = r.str();
    e.headers[k] = r.str();
  }
  uint64_t dn = r.u64();
  uint32_t np = r.u32();
  std::vector<uint64_t> ps(np);
  for (auto& p : ps) p = r.u64();
  size_t pos = r.pos();
  if (pos + dn > bytes.size()) throw CodecError("truncated envelope body");
  e.data.assign(bytes.substr(pos, dn));
  pos += dn;
  for (uint64_t n : ps) {
    if (pos + n > bytes.size()) throw CodecError("truncated envelope part");
    e.parts.emplace_back(bytes.substr(pos, n));
    pos += n;
  }
  return e;
}

}  // namespace mb
