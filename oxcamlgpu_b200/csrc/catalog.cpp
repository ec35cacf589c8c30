// Tile catalog: the host-side mirror of the reference's Gemm_catalog module
// (test/gemm_catalog.ml) and of the queries its emitter CLI answers
// (test/emit_gemm_ptx.ml:39-68).  Pure host C++; no CUDA here.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.hpp"

namespace oxgpu {

thread_local std::string g_last_error;

int fail(int status, const std::string &message) {
  g_last_error = message;
  return status;
}

// The ten entry symbols of examples/kernels/gemm.ml:165-199 and
// examples/kernels/gemm_bf16.ml:130-132, with the tile each was specialised
// for and the B200 variant that serves it.
static const CatalogEntry kEntries[] = {
    {"gemm_fast", {128, 256, 32, 4, 32}, 4, VARIANT_1CTA_128x256},
    {"gemm_bm128_bn256_s3", {128, 256, 32, 3, 32}, 4, VARIANT_1CTA_128x256},
    {"gemm_bm128_bn256_s2", {128, 256, 32, 2, 32}, 4, VARIANT_1CTA_128x256},
    {"gemm_bm128_bn128_s3", {128, 128, 32, 3, 32}, 4, VARIANT_1CTA_128x128},
    {"gemm_bm128_bn128_s2", {128, 128, 32, 2, 32}, 4, VARIANT_1CTA_128x128},
    {"gemm_bm64_bn256_s3", {64, 256, 32, 3, 32}, 4, VARIANT_1CTA_128x256},
    {"gemm_bm64_bn256_s2", {64, 256, 32, 2, 32}, 4, VARIANT_1CTA_128x256},
    {"gemm_bm256_bn128_s3", {256, 128, 32, 3, 32}, 4, VARIANT_1CTA_256x128},
    {"gemm_bm256_bn128_s2", {256, 128, 32, 2, 32}, 4, VARIANT_1CTA_256x128},
    {"gemm_bf16_fast", {128, 256, 64, 4, 32}, 2, VARIANT_1CTA_128x256},
};
static const int kEntryCount = (int)(sizeof(kEntries) / sizeof(kEntries[0]));

const CatalogEntry *find_entry(const char *name) {
  if (!name) return nullptr;
  for (int i = 0; i < kEntryCount; i++)
    if (std::strcmp(kEntries[i].name, name) == 0) return &kEntries[i];
  return nullptr;
}

// tile_catalog, test/gemm_catalog.ml:80-89 (order matters: entry 0 is the
// fallback tile).
static const oxgpu_tile_config kTileCatalog[] = {
    {128, 256, 32, 4, 32}, {128, 256, 32, 3, 32}, {128, 256, 32, 2, 32}, {128, 128, 32, 3, 32},
    {128, 128, 32, 2, 32}, {64, 256, 32, 3, 32},  {256, 128, 32, 3, 32},
};

static int threads_of(const oxgpu_tile_config &c) { return 128 * (c.bm / 64) + c.producers; }

// validate, test/gemm_catalog.ml:21-35: same checks in the same order, same
// messages.
static int validate(const oxgpu_tile_config &c) {
  if (c.bm % 64 != 0 || c.bm < 64)
    return fail(OXGPU_E_CONFIG, "BM must be a positive multiple of 64 (WGMMA m64)");
  if (!(c.bn >= 8 && c.bn <= 256 && c.bn % 8 == 0))
    return fail(OXGPU_E_CONFIG, "BN must be in {8,16,...,256} for WGMMA");
  if (c.bk % 32 != 0 || c.bk < 32 || c.bk > 32)
    return fail(OXGPU_E_CONFIG, "BK must be 32 (f32 TMA 128B swizzle box0 \xE2\x89\xA4 32)");
  if (c.stages < 2) return fail(OXGPU_E_CONFIG, "pipeline stages must be \xE2\x89\xA5 2");
  if (c.producers <= 0 || c.producers % 32 != 0)
    return fail(OXGPU_E_CONFIG, "producers must be a positive multiple of warp size (32)");
  if (threads_of(c) > 1024)
    return fail(OXGPU_E_CONFIG, "CTA threads (consumers+producers) must be \xE2\x89\xA4 1024");
  return OXGPU_OK;
}

static std::string trim(const std::string &s) {
  size_t b = 0, e = s.size();
  while (b < e && (s[b] == ' ' || s[b] == '\t' || s[b] == '\n' || s[b] == '\r' || s[b] == '\f'))
    b++;
  while (e > b && (s[e - 1] == ' ' || s[e - 1] == '\t' || s[e - 1] == '\n' ||
                   s[e - 1] == '\r' || s[e - 1] == '\f'))
    e--;
  return s.substr(b, e - b);
}

// OCaml's int_of_string_opt accepts an optional '-'/'+' sign, decimal digits
// with '_' separators, and 0x/0o/0b prefixes.  Catalog specs only ever use
// plain decimals; accept sign + decimal digits/underscores and the prefixed
// forms through strtol.
static bool parse_ocaml_int(const std::string &text, int *out) {
  if (text.empty()) return false;
  std::string digits;
  size_t i = 0;
  bool neg = false;
  if (text[0] == '-' || text[0] == '+') {
    neg = text[0] == '-';
    i = 1;
  }
  if (i >= text.size()) return false;
  int base = 10;
  if (text.size() > i + 1 && text[i] == '0') {
    char p = text[i + 1];
    if (p == 'x' || p == 'X') base = 16;
    else if (p == 'o' || p == 'O') base = 8;
    else if (p == 'b' || p == 'B') base = 2;
    if (base != 10) i += 2;
  }
  if (i >= text.size() || text[i] == '_') return false;
  for (; i < text.size(); i++) {
    char ch = text[i];
    if (ch == '_') continue;
    int v = (ch >= '0' && ch <= '9')   ? ch - '0'
            : (ch >= 'a' && ch <= 'f') ? ch - 'a' + 10
            : (ch >= 'A' && ch <= 'F') ? ch - 'A' + 10
                                       : 99;
    if (v >= base) return false;
    digits.push_back(ch);
  }
  if (digits.empty()) return false;
  long long v = std::strtoll(digits.c_str(), nullptr, base);
  if (digits.size() > 18 || v > 0x3fffffffffffffffLL) return false;
  if (v > 2147483647LL) return false;  // tile parameters are far below this
  *out = (int)(neg ? -v : v);
  return true;
}

// parse_config, test/gemm_catalog.ml:42-73.
static int parse_config(const char *spec, oxgpu_tile_config *out) {
  std::map<std::string, std::string> table;
  std::string s(spec);
  size_t start = 0;
  while (true) {
    size_t comma = s.find(',', start);
    std::string part = s.substr(start, comma == std::string::npos ? std::string::npos
                                                                    : comma - start);
    // String.split_on_char '=' must give exactly two pieces.
    size_t eq = part.find('=');
    if (eq == std::string::npos || part.find('=', eq + 1) != std::string::npos)
      return fail(OXGPU_E_CONFIG, "bad config fragment: " + part);
    table[trim(part.substr(0, eq))] = trim(part.substr(eq + 1));
    if (comma == std::string::npos) break;
    start = comma + 1;
  }
  auto integer = [&](const char *key, const std::string &text, int *v) -> int {
    if (!parse_ocaml_int(text, v))
      return fail(OXGPU_E_CONFIG,
                  std::string("config key ") + key + " is not an integer: " + text);
    return OXGPU_OK;
  };
  auto get = [&](const char *key, int *v) -> int {
    auto it = table.find(key);
    if (it == table.end()) return fail(OXGPU_E_CONFIG, std::string("missing config key: ") + key);
    return integer(key, it->second, v);
  };
  oxgpu_tile_config c{};
  int st;
  // The reference evaluates `stages` first, then the record fields; OCaml
  // evaluates record field expressions right to left, so a spec with several
  // faults reports producers, then bk, bn, bm.
  auto it = table.find("stages");
  if (it != table.end()) {
    if ((st = integer("stages", it->second, &c.stages))) return st;
  } else {
    c.stages = 3;
  }
  if ((st = get("producers", &c.producers))) return st;
  if ((st = get("bk", &c.bk))) return st;
  if ((st = get("bn", &c.bn))) return st;
  if ((st = get("bm", &c.bm))) return st;
  if ((st = validate(c))) return st;
  *out = c;
  return OXGPU_OK;
}

// ---- .gpu metadata header (lib/frontend/gpu_metadata.ml, format 3) ---------------
static std::vector<std::string> split(const std::string &s, char sep) {
  std::vector<std::string> out;
  size_t start = 0;
  while (true) {
    size_t pos = s.find(sep, start);
    out.push_back(s.substr(start, pos == std::string::npos ? std::string::npos : pos - start));
    if (pos == std::string::npos) break;
    start = pos + 1;
  }
  return out;
}

// `integer` / `id` (gpu_metadata.ml:12-18)
static int meta_integer(const std::string &text, int *v) {
  if (!parse_ocaml_int(text, v)) return fail(OXGPU_E_CONFIG, "invalid integer " + text);
  return OXGPU_OK;
}
static int meta_id(const std::string &text, int *v) {
  int st = meta_integer(text, v);
  if (st) return st;
  if (*v < 0) return fail(OXGPU_E_CONFIG, "negative value/argument id");
  return OXGPU_OK;
}

// `parse_slot` (gpu_metadata.ml:130-159): type, ownership, locality,
// portability, permission, then the source span (quoted file, four numbers).
static int parse_slot(const std::vector<std::string> &f, size_t from, oxgpu_gpu_slot *out) {
  if (f.size() - from != 10) return fail(OXGPU_E_CONFIG, "missing or extra mode fields");
  const std::string &file = f[from + 5];
  if (file.size() < 2 || file.front() != '"' || file.back() != '"')
    return fail(OXGPU_E_CONFIG, "invalid source filename");
  int st;
  if ((st = meta_id(f[from + 6], &out->start_line)) || (st = meta_id(f[from + 7], &out->start_col)) ||
      (st = meta_id(f[from + 8], &out->end_line)) || (st = meta_id(f[from + 9], &out->end_col)))
    return st;
  static const char *types[] = {"scalar_i32", "scalar_f32", "bool", "unit", "buffer_f32",
                                "buffer_bf16", "buffer_f16", "tensor_map", "scalar_u64"};
  out->type = 0;
  for (int i = 0; i < 9; i++)
    if (f[from] == types[i]) out->type = i + 1;
  if (!out->type) return fail(OXGPU_E_CONFIG, "unsupported frontend type");
  const std::string &o = f[from + 1], &l = f[from + 2], &p = f[from + 3], &a = f[from + 4];
  out->ownership = o == "unique" ? OXGPU_OWN_UNIQUE : o == "aliased" ? OXGPU_OWN_ALIASED : 0;
  if (!out->ownership) return fail(OXGPU_E_CONFIG, "invalid ownership");
  out->locality = l == "local" ? OXGPU_LOC_LOCAL : l == "global" ? OXGPU_LOC_GLOBAL : 0;
  if (!out->locality) return fail(OXGPU_E_CONFIG, "invalid locality");
  out->portability = p == "portable" ? OXGPU_PORT_PORTABLE : p == "nonportable" ? OXGPU_PORT_NONPORTABLE
                     : p == "unspecified" ? OXGPU_PORT_UNSPECIFIED : 0;
  if (!out->portability) return fail(OXGPU_E_CONFIG, "invalid portability");
  out->permission = a == "read" ? OXGPU_PERM_READ : a == "write" ? OXGPU_PERM_WRITE
                    : a == "read_write" ? OXGPU_PERM_READ_WRITE : a == "immutable" ? OXGPU_PERM_IMMUTABLE : 0;
  if (!out->permission) return fail(OXGPU_E_CONFIG, "invalid permission");
  return OXGPU_OK;
}

// header part of `parse` (gpu_metadata.ml:289-343)
static int parse_gpu_header(const std::string &source, oxgpu_gpu_header *out) {
  std::vector<std::string> lines;
  for (auto &line : split(source, '\n'))
    if (!line.empty()) lines.push_back(line);  // blank lines are dropped before parsing
  size_t pos = 0;
  auto peek = [&]() { return pos == lines.size() ? std::vector<std::string>() : split(lines[pos], '\t'); };
  std::memset(out, 0, sizeof *out);
  {
    auto row = peek();
    pos++;
    if (row.size() != 2 || row[0] != "format" || row[1] != "3")
      return fail(OXGPU_E_CONFIG, "malformed region/header");
  }
  {
    auto row = peek();
    pos++;
    if (row.size() != 2 || row[0] != "kernel" || row[1].empty()) return fail(OXGPU_E_CONFIG, "missing kernel");
    if (row[1].size() >= sizeof out->kernel) return fail(OXGPU_E_TOO_LARGE, "kernel name too long");
    std::strcpy(out->kernel, row[1].c_str());
  }
  {
    auto row = peek();
    if (row.size() == 2 && row[0] == "threads") {
      pos++;
      int st = meta_integer(row[1], &out->threads);
      if (st) return st;
      if (out->threads < 1 || out->threads > 1024)
        return fail(OXGPU_E_CONFIG, "CTA thread count must be in 1..1024");
    }
  }
  while (true) {
    auto row = peek();
    if (row.size() < 2 || row[0] != "arg") break;
    pos++;
    int index, st;
    if ((st = meta_id(row[1], &index))) return st;
    if (index != out->nargs) return fail(OXGPU_E_CONFIG, "argument ids must be contiguous");
    if (out->nargs >= 16) return fail(OXGPU_E_TOO_LARGE, "more than 16 kernel arguments");
    if ((st = parse_slot(row, 2, &out->args[out->nargs]))) return st;
    out->nargs++;
  }
  {
    auto row = peek();
    if (row.empty() || row[0] != "result") return fail(OXGPU_E_CONFIG, "missing result");
    int st = parse_slot(row, 1, &out->result);
    if (st) return st;
  }
  return OXGPU_OK;
}

}  // namespace oxgpu

using namespace oxgpu;

extern "C" {

const char *oxgpu_b200_last_error(void) { return g_last_error.c_str(); }

const char *oxgpu_b200_strerror(int status) {
  switch (status) {
    case OXGPU_OK: return "ok";
    case OXGPU_E_INVALID_ARG: return "invalid argument";
    case OXGPU_E_CONFIG: return "tile configuration rejected";
    case OXGPU_E_UNKNOWN_KERNEL: return "no such kernel in the catalog";
    case OXGPU_E_SHAPE: return "problem size not divisible by the tile";
    case OXGPU_E_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case OXGPU_E_TOO_LARGE: return "size exceeds a documented maximum";
    case OXGPU_E_DEVICE_TIMEOUT: return "a bounded device-side wait timed out";
    case OXGPU_E_NO_DRIVER: return "CUDA driver entry point unavailable";
    default: return status > 0 ? "CUDA error" : "unknown status";
  }
}

int oxgpu_b200_config_threads(const oxgpu_tile_config *c) {
  if (!c) return fail(OXGPU_E_INVALID_ARG, "config is null");
  return threads_of(*c);
}

int oxgpu_b200_validate_config(const oxgpu_tile_config *c) {
  if (!c) return fail(OXGPU_E_INVALID_ARG, "config is null");
  return validate(*c);
}

int oxgpu_b200_string_of_config(const oxgpu_tile_config *c, char *buf, size_t cap) {
  if (!c || !buf || cap == 0) return fail(OXGPU_E_INVALID_ARG, "null argument");
  int n = std::snprintf(buf, cap, "bm=%d,bn=%d,bk=%d,stages=%d,producers=%d,threads=%d", c->bm,
                        c->bn, c->bk, c->stages, c->producers, threads_of(*c));
  if (n < 0 || (size_t)n >= cap) return fail(OXGPU_E_TOO_LARGE, "buffer too small");
  return OXGPU_OK;
}

int oxgpu_b200_parse_config(const char *spec, oxgpu_tile_config *out) {
  if (!spec || !out) return fail(OXGPU_E_INVALID_ARG, "null argument");
  return parse_config(spec, out);
}

int oxgpu_b200_catalog_size(void) { return (int)(sizeof(kTileCatalog) / sizeof(kTileCatalog[0])); }

int oxgpu_b200_catalog_get(int index, oxgpu_tile_config *out) {
  if (!out || index < 0 || index >= oxgpu_b200_catalog_size())
    return fail(OXGPU_E_INVALID_ARG, "catalog index out of range");
  *out = kTileCatalog[index];
  return OXGPU_OK;
}

// kernel_binding, test/gemm_catalog.ml:101-112.  The match is on the f32
// tiles only (bk = 32); gemm_bf16_fast is reached by name, as in the
// reference's bench driver (bench/run.sh:104).
int oxgpu_b200_kernel_binding(const oxgpu_tile_config *c, const char **name) {
  if (!c || !name) return fail(OXGPU_E_INVALID_ARG, "null argument");
  for (int i = 0; i < kEntryCount; i++) {
    const CatalogEntry &e = kEntries[i];
    if (e.element_bytes != 4) continue;
    if (e.tile.bm == c->bm && e.tile.bn == c->bn && e.tile.bk == c->bk &&
        e.tile.stages == c->stages && e.tile.producers == c->producers) {
      *name = e.name;
      return OXGPU_OK;
    }
  }
  char text[160];
  std::snprintf(text, sizeof text, "bm=%d,bn=%d,bk=%d,stages=%d,producers=%d,threads=%d", c->bm,
                c->bn, c->bk, c->stages, c->producers, threads_of(*c));
  return fail(OXGPU_E_UNKNOWN_KERNEL, std::string("no OxCaml kernel for ") + text);
}

// choose_config, test/gemm_catalog.ml:114-137: the aspect ratio picks the tile,
// K is accepted and unused.
int oxgpu_b200_choose_config(int m, int n, int k, oxgpu_tile_config *out) {
  (void)k;
  if (!out) return fail(OXGPU_E_INVALID_ARG, "null argument");
  oxgpu_tile_config c;
  if (m >= 2 * n) c = {256, 128, 32, 3, 32};
  else if (m <= 1024 && n <= 1024 && m < 2 * n && n < 2 * m) c = {64, 256, 32, 3, 32};
  else c = {128, 256, 32, 4, 32};
  int st = validate(c);
  if (st) return st;
  *out = c;
  return OXGPU_OK;
}

int oxgpu_b200_kernel_tile(const char *name, oxgpu_tile_config *tile, int *element_bytes) {
  const CatalogEntry *e = find_entry(name);
  if (!e) return fail(OXGPU_E_UNKNOWN_KERNEL, std::string("no kernel named ") + (name ? name : "(null)"));
  if (tile) *tile = e->tile;
  if (element_bytes) *element_bytes = e->element_bytes;
  return OXGPU_OK;
}

int oxgpu_b200_kernel_info(const char *name, int *threads, int *dynamic_smem, int *total_smem) {
  const CatalogEntry *e = find_entry(name);
  if (!e) return fail(OXGPU_E_UNKNOWN_KERNEL, std::string("no kernel named ") + (name ? name : "(null)"));
  int smem = variant_smem_bytes(e->variant, e->tile.stages);
  if (threads) *threads = kThreadsPerCta;
  if (dynamic_smem) *dynamic_smem = smem;
  if (total_smem) *total_smem = smem;
  return OXGPU_OK;
}

int oxgpu_b200_parse_gpu_header(const char *text, size_t length, oxgpu_gpu_header *out) {
  if (!text || !out) return fail(OXGPU_E_INVALID_ARG, "null argument");
  return parse_gpu_header(std::string(text, length), out);
}

int oxgpu_b200_check_gpu_header(const oxgpu_gpu_header *h) {
  if (!h) return fail(OXGPU_E_INVALID_ARG, "null argument");
  const CatalogEntry *e = find_entry(h->kernel);
  if (!e) return fail(OXGPU_E_UNKNOWN_KERNEL, std::string("no kernel named ") + h->kernel);
  const int want_threads = threads_of(e->tile);
  if (h->threads != want_threads) {
    char text[160];
    std::snprintf(text, sizeof text, "%s is specialised for %d threads per CTA, the metadata says %d",
                  h->kernel, want_threads, h->threads);
    return fail(OXGPU_E_CONFIG, text);
  }
  if (h->nargs != 6) return fail(OXGPU_E_CONFIG, "a GEMM entry point takes six arguments (a_tmap, b_tmap, c, m, n, k)");
  for (int i = 0; i < 2; i++) {
    const oxgpu_gpu_slot &s = h->args[i];
    if (s.type != OXGPU_TY_TENSOR_MAP || s.ownership != OXGPU_OWN_ALIASED || s.permission != OXGPU_PERM_READ)
      return fail(OXGPU_E_CONFIG, "arguments 0 and 1 must be tensor maps, aliased and read-only");
  }
  const oxgpu_gpu_slot &c = h->args[2];
  if (c.type != OXGPU_TY_BUFFER_F32 || c.ownership != OXGPU_OWN_UNIQUE || c.permission != OXGPU_PERM_READ_WRITE)
    return fail(OXGPU_E_CONFIG, "argument 2 must be the f32 output buffer, unique and read_write");
  for (int i = 3; i < 6; i++)
    if (h->args[i].type != OXGPU_TY_SCALAR_I32)
      return fail(OXGPU_E_CONFIG, "arguments 3 to 5 must be i32 scalars (m, n, k)");
  return OXGPU_OK;
}

// Grouped CTA order, tools/exporter/export_prims_index.ml:52-58.
int oxgpu_b200_grouped_tile(int pid, int group, int tiles_m, int tiles_n, int *tile_m,
                            int *tile_n) {
  if (!tile_m || !tile_n || group <= 0 || tiles_m <= 0 || tiles_n <= 0 || pid < 0 ||
      (long long)pid >= (long long)tiles_m * tiles_n)
    return fail(OXGPU_E_INVALID_ARG, "grouped_tile: argument out of range");
  grouped_tile(pid, group, tiles_m, tiles_n, tile_m, tile_n);
  return OXGPU_OK;
}

// The kernels' own walk: grouped_tile with the columns of every other group of
// tile rows reversed, through the reciprocal arithmetic the kernels use.
int oxgpu_b200_tile_walk(int pid, int group, int tiles_m, int tiles_n, int *tile_m, int *tile_n) {
  if (!tile_m || !tile_n || group <= 0 || tiles_m <= 0 || tiles_n <= 0 || pid < 0 ||
      (long long)pid >= (long long)tiles_m * tiles_n || (long long)group * tiles_n > 0x7fffffffLL)
    return fail(OXGPU_E_INVALID_ARG, "tile_walk: argument out of range");
  const long long work = (long long)tiles_m * tiles_n;
  const FastDivisor per_group = make_fast_divisor(group * tiles_n, work), by_group = make_fast_divisor(group, work);
  int group_index;
  grouped_tile_fast(pid, per_group, by_group, tiles_m, tile_m, tile_n, &group_index);
  if (group_index & 1) *tile_n = tiles_n - 1 - *tile_n;
  return OXGPU_OK;
}

}  // extern "C"
