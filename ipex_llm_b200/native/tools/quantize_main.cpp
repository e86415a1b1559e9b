// ipex-quantize: rewrite a GGUF file with its large matrices packed into a k-quant super-block format.
//
// The reference ships prebuilt `quantize-<family>` executables that turn an fp16 ggml file into a low-bit one
// (python/llm/src/ipex_llm/ggml/quantize.py:87-142 shells out to them).  This is the counterpart for the container
// format in use today: it streams a GGUF v2/v3 file, keeps the metadata section byte for byte, packs every 2-D
// f32 / f16 / bf16 tensor whose row length is a multiple of 256 with the quantizers of quant_core (q2_k, q4_k, q5_k,
// q6_k: ggml super-block layouts), copies everything else unchanged, and writes a GGUF file any GGUF reader opens.
//
//   ipex-quantize <in.gguf> <out.gguf> <q2_k|q4_k|q5_k|q6_k> [--keep <substring>]... [--output-type <type>]
//
// `--keep` leaves tensors whose name contains the substring untouched; `--output-type` gives `output.weight` and
// `token_embd.weight` their own format (q6_k by default when the body is q2_k / q4_k, as is customary for those files).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../host/quant_core.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
enum GgmlType : uint32_t { T_F32 = 0, T_F16 = 1, T_Q2_K = 10, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30 };

// Every count and length of the file is checked against the bytes that are left, so a truncated or corrupt file ends
// in an error message instead of a huge allocation or a loop over billions of absent entries.
struct Reader {
  FILE* f;
  uint64_t size = 0;
  bool ok = true;
  uint64_t left() const { long p = ftell(f); return p < 0 || (uint64_t)p > size ? 0 : size - (uint64_t)p; }
  template <typename T> T get() {
    T v{};
    if (fread(&v, sizeof(T), 1, f) != 1) ok = false;
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    std::string s;
    if (!ok || n > left()) { ok = false; return s; }
    s.resize(n);
    if (n && fread(&s[0], 1, n, f) != n) ok = false;
    return s;
  }
  void skip(uint64_t n) { if (n > left() || fseek(f, (long)n, SEEK_CUR) != 0) ok = false; }
};

// bytes of one scalar GGUF metadata value type (0 for string / array)
size_t scalar_size(uint32_t t) {
  switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}

bool skip_value(Reader& r, uint32_t t, uint32_t* u32_out) {
  if (t == 8) { r.str(); return r.ok; }
  if (t == 9) {
    uint32_t et = r.get<uint32_t>();
    uint64_t n = r.get<uint64_t>();
    if (!r.ok) return false;
    if (et == 8) {
      if (n > r.left() / 8) return false;                  // every string carries an 8-byte length
      for (uint64_t i = 0; i < n && r.ok; i++) r.str();
      return r.ok;
    }
    size_t sz = scalar_size(et);
    if (!sz || n > r.left() / sz) return false;
    r.skip(n * sz);
    return r.ok;
  }
  size_t sz = scalar_size(t);
  if (!sz) return false;
  if (t == 4 && u32_out) { *u32_out = r.get<uint32_t>(); return r.ok; }
  r.skip(sz);
  return r.ok;
}

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> dims;
  uint32_t type = 0;
  uint64_t offset = 0;   // relative to the data section
  uint64_t nbytes = 0;
  // output side
  uint32_t out_type = 0;
  int out_core = 0;      // quant_core id of out_type when the tensor is re-packed
  uint64_t out_offset = 0, out_nbytes = 0;
};

bool type_geometry(uint32_t t, int* qk, int* ts) {
  switch (t) {
    case T_F32: *qk = 1; *ts = 4; return true;
    case T_F16: case T_BF16: *qk = 1; *ts = 2; return true;
    case 2: *qk = 32; *ts = 18; return true;   // q4_0
    case 3: *qk = 32; *ts = 20; return true;   // q4_1
    case 6: *qk = 32; *ts = 22; return true;   // q5_0
    case 7: *qk = 32; *ts = 24; return true;   // q5_1
    case 8: *qk = 32; *ts = 34; return true;   // q8_0
    case T_Q2_K: *qk = 256; *ts = 84; return true;
    case 11: *qk = 256; *ts = 110; return true;  // q3_k
    case T_Q4_K: *qk = 256; *ts = 144; return true;
    case T_Q5_K: *qk = 256; *ts = 176; return true;
    case T_Q6_K: *qk = 256; *ts = 210; return true;
    case 16: *qk = 256; *ts = 66; return true;   // iq2_xxs
    case 17: *qk = 256; *ts = 74; return true;   // iq2_xs
    case 19: *qk = 256; *ts = 50; return true;   // iq1_s
    case 29: *qk = 256; *ts = 56; return true;   // iq1_m
    default: return false;
  }
}

bool parse_target(const char* s, uint32_t* ggml, int* core) {
  if (!strcmp(s, "q2_k")) { *ggml = T_Q2_K; *core = QT_Q2_K; return true; }
  if (!strcmp(s, "q4_k")) { *ggml = T_Q4_K; *core = QT_Q4_K; return true; }
  if (!strcmp(s, "q5_k")) { *ggml = T_Q5_K; *core = QT_Q5_K; return true; }
  if (!strcmp(s, "q6_k")) { *ggml = T_Q6_K; *core = QT_Q6_K; return true; }
  return false;
}

float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

int fail(const char* msg) { fprintf(stderr, "ipex-quantize: %s\n", msg); return 1; }

}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) {
    fprintf(stderr, "usage: %s <in.gguf> <out.gguf> <q2_k|q4_k|q5_k|q6_k> [--keep <substr>]... [--output-type <type>]\n",
            argv[0]);
    return 2;
  }
  uint32_t body_ggml; int body_core;
  if (!parse_target(argv[3], &body_ggml, &body_core)) return fail("unknown target format");
  uint32_t head_ggml = body_ggml; int head_core = body_core;
  if (body_ggml == T_Q2_K || body_ggml == T_Q4_K) { head_ggml = T_Q6_K; head_core = QT_Q6_K; }
  std::vector<std::string> keep;
  for (int i = 4; i < argc; i++) {
    if (!strcmp(argv[i], "--keep") && i + 1 < argc) keep.push_back(argv[++i]);
    else if (!strcmp(argv[i], "--output-type") && i + 1 < argc) {
      if (!parse_target(argv[++i], &head_ggml, &head_core)) return fail("unknown --output-type");
    } else return fail("unknown argument");
  }

  FILE* in = fopen(argv[1], "rb");
  if (!in) return fail("cannot open the input file");
  Reader r{in};
  fseek(in, 0, SEEK_END);
  r.size = (uint64_t)ftell(in);
  fseek(in, 0, SEEK_SET);
  if (r.get<uint32_t>() != kMagic) return fail("not a GGUF file");
  uint32_t version = r.get<uint32_t>();
  if (version != 2 && version != 3) return fail("unsupported GGUF version");
  uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  // a metadata entry takes at least 13 bytes (key length, type, one byte), a tensor entry at least 24
  if (!r.ok || n_kv > r.left() / 13 || n_tensors > r.left() / 24) return fail("malformed header");
  long kv_begin = ftell(in);
  uint32_t alignment = 32;
  for (uint64_t i = 0; i < n_kv; i++) {
    std::string key = r.str();
    uint32_t t = r.get<uint32_t>();
    uint32_t u = 0;
    if (!r.ok || !skip_value(r, t, &u)) return fail("malformed metadata section");
    if (key == "general.alignment" && t == 4 && u) alignment = u;
  }
  long kv_end = ftell(in);
  std::vector<TensorInfo> infos(n_tensors);
  for (auto& ti : infos) {
    ti.name = r.str();
    uint32_t nd = r.get<uint32_t>();
    if (!r.ok || nd > 8) return fail("malformed tensor table");
    ti.dims.resize(nd);
    for (auto& d : ti.dims) d = r.get<uint64_t>();
    ti.type = r.get<uint32_t>();
    ti.offset = r.get<uint64_t>();
    int qk, ts;
    if (!r.ok || !type_geometry(ti.type, &qk, &ts)) return fail("tensor of an unknown ggml type");
    uint64_t n = 1;
    for (auto d : ti.dims) {
      // no format stores less than one bit per element: more elements than bits in the file cannot be real
      if (d == 0 || n > r.size * 8 / d) return fail("tensor larger than the file");  // (also guards the product)
      n *= d;
    }
    ti.nbytes = n / qk * ts;
  }
  if (alignment == 0 || alignment > (1u << 20)) return fail("implausible general.alignment");
  uint64_t data_start = align_up((uint64_t)ftell(in), alignment);
  for (auto& ti : infos)
    if (ti.offset > r.size || ti.nbytes > r.size || data_start + ti.offset + ti.nbytes > r.size)
      return fail("tensor data reaches beyond the end of the file");

  // decide the output type of every tensor and lay the output data section out
  uint64_t off = 0;
  for (auto& ti : infos) {
    ti.out_type = ti.type;
    ti.out_nbytes = ti.nbytes;
    bool dense = ti.type == T_F32 || ti.type == T_F16 || ti.type == T_BF16;
    bool kept = false;
    for (auto& k : keep) kept = kept || ti.name.find(k) != std::string::npos;
    if (dense && !kept && ti.dims.size() == 2 && ti.dims[0] % 256 == 0) {
      bool head = ti.name == "output.weight" || ti.name == "token_embd.weight";
      ti.out_type = head ? head_ggml : body_ggml;
      ti.out_core = head ? head_core : body_core;
      int qk, ts;
      type_geometry(ti.out_type, &qk, &ts);
      ti.out_nbytes = ti.dims[0] * ti.dims[1] / qk * ts;
    }
    ti.out_offset = off;
    off = align_up(off + ti.out_nbytes, alignment);
  }

  FILE* out = fopen(argv[2], "wb");
  if (!out) return fail("cannot open the output file");
  auto put = [&](const void* p, size_t n) { return fwrite(p, 1, n, out) == n; };
  uint32_t magic = kMagic;
  bool ok = put(&magic, 4) && put(&version, 4) && put(&n_tensors, 8) && put(&n_kv, 8);
  {  // metadata, verbatim
    std::vector<char> kv((size_t)(kv_end - kv_begin));
    fseek(in, kv_begin, SEEK_SET);
    if (!kv.empty() && fread(kv.data(), 1, kv.size(), in) != kv.size()) return fail("short read");
    ok = ok && put(kv.data(), kv.size());
  }
  for (auto& ti : infos) {
    uint64_t len = ti.name.size();
    uint32_t nd = (uint32_t)ti.dims.size();
    ok = ok && put(&len, 8) && put(ti.name.data(), len) && put(&nd, 4);
    for (auto d : ti.dims) ok = ok && put(&d, 8);
    ok = ok && put(&ti.out_type, 4) && put(&ti.out_offset, 8);
  }
  uint64_t pos = (uint64_t)ftell(out);
  std::vector<char> zeros(alignment, 0);
  ok = ok && put(zeros.data(), (size_t)(align_up(pos, alignment) - pos));
  uint64_t out_data_start = align_up(pos, alignment);

  std::vector<char> raw;
  std::vector<float> f32;
  std::vector<char> packed;
  size_t n_packed = 0;
  for (auto& ti : infos) {
    raw.resize(ti.nbytes);
    fseek(in, (long)(data_start + ti.offset), SEEK_SET);
    if (ti.nbytes && fread(raw.data(), 1, ti.nbytes, in) != ti.nbytes) return fail("short read in the data section");
    uint64_t here = (uint64_t)ftell(out) - out_data_start;
    if (here > ti.out_offset) return fail("internal layout error");
    for (uint64_t gap = ti.out_offset - here; gap > 0;) {
      size_t step = (size_t)(gap < alignment ? gap : alignment);
      ok = ok && put(zeros.data(), step);
      gap -= step;
    }
    if (ti.out_type == ti.type) {
      ok = ok && put(raw.data(), raw.size());
      continue;
    }
    uint64_t n = ti.dims[0] * ti.dims[1];
    f32.resize(n);
    if (ti.type == T_F32) memcpy(f32.data(), raw.data(), n * 4);
    else if (ti.type == T_F16) {
      const uint16_t* h = (const uint16_t*)raw.data();
      for (uint64_t i = 0; i < n; i++) f32[i] = half_to_float(h[i]);
    } else {
      const uint16_t* h = (const uint16_t*)raw.data();
      for (uint64_t i = 0; i < n; i++) { uint32_t b = (uint32_t)h[i] << 16; memcpy(&f32[i], &b, 4); }
    }
    packed.resize(ti.out_nbytes);
    size_t wrote = ggml_quantize_tensor(f32.data(), packed.data(), ti.out_core, (size_t)n, (int)ti.dims[0], nullptr, 0);
    if (wrote != ti.out_nbytes) return fail("quantizer wrote an unexpected number of bytes");
    ok = ok && put(packed.data(), packed.size());
    n_packed++;
  }
  uint64_t end = (uint64_t)ftell(out) - out_data_start;
  ok = ok && put(zeros.data(), (size_t)(align_up(end, alignment) - end));
  fclose(in);
  if (fclose(out) != 0 || !ok) return fail("write failed");
  printf("ipex-quantize: %zu of %zu tensors packed to %s\n", n_packed, infos.size(), argv[3]);
  return 0;
}
