// see-cuda-plan-probe — runs one section of a sealed .seeu plan on the CUDA
// backend against a caller-supplied arena image, through the C ABI
// (include/see_cuda.h) and nothing else.  It speaks the command line and the
// file formats of the reference's seeml-plan-probe (reference:
// tool/seeml_plan_probe.cc:534-700; trace container tool/probe_trace.h), so the
// reference's own differ (tool/frontier_exec.py diff --probe <this>) can drive
// this backend as it drives the CPU one:
//
//   --plan P --section train|eval|merge|step --arena-in IMG --arena-out IMG
//   --lr-bits HEXF32 --step N [--source MODEL] [--backend NAME] [--threads N]
//   one of:  (nothing)   execute once
//            --trace F   execute once, flushing after every instruction, and
//                        record every extent the instruction may write
//            --time N    one warm-up, then N flushed executions; one JSON line
//            --profile N per-opcode wall time over N executions; one JSON line
//
// --backend and --threads are accepted and ignored (there is one backend here;
// the differ passes "cpu").  Exit 0 with --arena-out written, or 1 with a
// one-line diagnostic on stderr.
#include <algorithm>
#include <chrono>
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <vector>

#include "../../include/see_cuda.h"
#include "extents.h"
#include "plan_abi.h"

namespace {

int Fail(const std::string& why) {
  std::fprintf(stderr, "see-cuda-plan-probe: %s\n", why.c_str());
  return 1;
}

bool ReadWhole(const std::string& path, std::vector<uint8_t>* out) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) return false;
  const std::streamsize n = f.tellg();
  if (n < 0) return false;
  out->resize(static_cast<size_t>(n));
  f.seekg(0);
  return n == 0 || static_cast<bool>(f.read(reinterpret_cast<char*>(out->data()), n));
}

bool WriteWhole(const std::string& path, const void* data, size_t bytes) {
  const std::string tmp = path + ".partial";
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) return false;
    f.write(static_cast<const char*>(data), static_cast<std::streamsize>(bytes));
    if (!f) return false;
  }
  return std::rename(tmp.c_str(), path.c_str()) == 0;
}

template <typename T>
void Put(std::vector<uint8_t>* buf, T v) {
  const auto* p = reinterpret_cast<const uint8_t*>(&v);
  buf->insert(buf->end(), p, p + sizeof(T));
}

struct Options {
  std::string plan, section = "train", arena_in, arena_out, trace, source;
  uint32_t lr_bits = 0;
  uint64_t step = 1, timed = 0, profiled = 0;
};

}  // namespace

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto value = [&](std::string* dst) {
      if (i + 1 >= argc) return false;
      *dst = argv[++i];
      return true;
    };
    std::string v;
    if (a == "--version") { std::printf("see-cuda-plan-probe 1\n"); return 0; }
    else if (a == "--plan") { if (!value(&o.plan)) return Fail("--plan wants a path"); }
    else if (a == "--section") { if (!value(&o.section)) return Fail("--section wants a name"); }
    else if (a == "--arena-in") { if (!value(&o.arena_in)) return Fail("--arena-in wants a path"); }
    else if (a == "--arena-out") { if (!value(&o.arena_out)) return Fail("--arena-out wants a path"); }
    else if (a == "--trace") { if (!value(&o.trace)) return Fail("--trace wants a path"); }
    else if (a == "--source") { if (!value(&o.source)) return Fail("--source wants a path"); }
    else if (a == "--backend" || a == "--threads") { if (!value(&v)) return Fail(a + " wants a value"); }
    else if (a == "--lr-bits") { if (!value(&v)) return Fail("--lr-bits wants a hex float"); o.lr_bits = static_cast<uint32_t>(std::strtoul(v.c_str(), nullptr, 16)); }
    else if (a == "--step") { if (!value(&v)) return Fail("--step wants a number"); o.step = std::strtoull(v.c_str(), nullptr, 10); }
    else if (a == "--time") { if (!value(&v)) return Fail("--time wants a count"); o.timed = std::strtoull(v.c_str(), nullptr, 10); }
    else if (a == "--profile") { if (!value(&v)) return Fail("--profile wants a count"); o.profiled = std::strtoull(v.c_str(), nullptr, 10); }
    else return Fail("unknown argument '" + a + "'");
  }
  if (o.plan.empty() || o.arena_in.empty() || o.arena_out.empty())
    return Fail("usage: --plan P --section S --arena-in IMG --arena-out IMG [--trace F | --time N | --profile N] "
                "--lr-bits HEX --step N [--source MODEL]");
  if (o.section != "train" && o.section != "eval" && o.section != "merge" && o.section != "step")
    return Fail("--section is one of train, eval, merge, step");
  if ((!o.trace.empty()) + (o.timed != 0) + (o.profiled != 0) > 1)
    return Fail("--trace, --time and --profile exclude each other");

  std::vector<uint8_t> plan;
  if (!ReadWhole(o.plan, &plan)) return Fail("cannot read the plan");
  if (plan.size() < sizeof(see::PlanHeader)) return Fail("the plan is truncated");
  see::PlanHeader h;
  std::memcpy(&h, plan.data(), sizeof(h));
  if (h.magic != see::kSeeuMagic) return Fail("not a .seeu plan");
  uint64_t off = h.train_instr_offset, count = h.train_instr_count;
  if (o.section == "eval") off = h.eval_instr_offset, count = h.eval_instr_count;
  if (o.section == "merge") off = h.merge_instr_offset, count = h.merge_instr_count;
  if (o.section == "step") off = h.step_instr_offset, count = h.step_instr_count;
  if (count > plan.size() / sizeof(see::Instruction) || off > plan.size() ||
      count * sizeof(see::Instruction) > plan.size() - off || h.rodata_offset > plan.size() ||
      h.rodata_size > plan.size() - h.rodata_offset)
    return Fail("a plan section lies outside the file");
  std::vector<see::Instruction> program(count);
  if (count) std::memcpy(program.data(), plan.data() + off, count * sizeof(see::Instruction));

  std::vector<uint8_t> source;
  if (!o.source.empty() && !ReadWhole(o.source, &source)) return Fail("cannot read --source");
  std::vector<see::Extents> extents(count);
  for (size_t i = 0; i < count; ++i) {
    const std::string e = see::DescribeInstruction(program[i], h.arena_size, h.rodata_size, source.size(), &extents[i]);
    if (!e.empty()) return Fail("instruction " + std::to_string(i) + ": " + e);
  }

  const size_t aligned = std::max<size_t>(1, (h.arena_size + see::kArenaAlignment - 1) / see::kArenaAlignment) *
                         see::kArenaAlignment;
  std::vector<uint8_t> image;
  if (!ReadWhole(o.arena_in, &image)) return Fail("cannot read the arena image");
  if (image.size() != h.arena_size)
    return Fail("the arena image is " + std::to_string(image.size()) + " bytes; the plan declares " +
                std::to_string(h.arena_size));
  image.resize(aligned, 0);

  see_cuda_backend* be = nullptr;
  if (see_cuda_create(0, &be) != SEE_OK) return Fail(see_cuda_create_error());
  auto fail_be = [&](const char* what) {
    const std::string msg = std::string(what) + ": " + see_cuda_last_error(be);
    see_cuda_destroy(be);
    return Fail(msg);
  };
  if (see_cuda_bind(be, image.data(), aligned, plan.data() + h.rodata_offset, h.rodata_size) != SEE_OK)
    return fail_be("bind");
  if (!source.empty() && see_cuda_bind_source(be, source.data(), source.size()) != SEE_OK)
    return fail_be("bind source");

  see_step_params params{};
  std::memcpy(&params.lr, &o.lr_bits, 4);
  params.beta1 = h.beta1; params.beta2 = h.beta2; params.eps = h.eps; params.weight_decay = h.weight_decay;
  params.step = o.step;
  auto counters = [&] {
    see_cuda_counters c{};
    see_cuda_counters_get(be, &c);
    return c;
  };
  using Clock = std::chrono::steady_clock;
  auto run_all = [&]() -> int {   // every instruction of the section, then a flush; -1 or the failing index + 1
    for (size_t i = 0; i < count; ++i)
      if (see_cuda_execute(be, &program[i], &params) != SEE_OK) return static_cast<int>(i) + 1;
    return see_cuda_flush(be) == SEE_OK ? 0 : -1;
  };

  if (o.timed) {
    std::vector<double> ms;
    uint64_t relaxed0 = 0;
    for (uint64_t run = 0; run <= o.timed; ++run) {   // run 0 warms up
      const auto t0 = Clock::now();
      if (const int rc = run_all(); rc != 0) return fail_be(rc > 0 ? "execute" : "flush");
      if (run) ms.push_back(std::chrono::duration<double, std::milli>(Clock::now() - t0).count());
      else relaxed0 = counters().relaxed_executions;
    }
    std::sort(ms.begin(), ms.end());
    const size_t n = ms.size();
    std::printf("{\"backend\": \"%s\", \"section\": \"%s\", \"executions\": %zu, \"ms_median\": %.4f, "
                "\"ms_min\": %.4f, \"ms_max\": %.4f, \"relaxed_executions\": %" PRIu64 "}\n",
                see_cuda_name(be), o.section.c_str(), n, n % 2 ? ms[n / 2] : 0.5 * (ms[n / 2 - 1] + ms[n / 2]),
                ms.front(), ms.back(), counters().relaxed_executions - relaxed0);
  } else if (o.profiled) {
    std::map<std::string, std::pair<double, uint64_t>> rows;
    double total = 0.0;
    uint64_t relaxed0 = 0;
    for (uint64_t run = 0; run <= o.profiled; ++run) {
      if (run == 1) relaxed0 = counters().relaxed_executions;
      for (size_t i = 0; i < count; ++i) {
        const auto t0 = Clock::now();
        if (see_cuda_execute(be, &program[i], &params) != SEE_OK || see_cuda_flush(be) != SEE_OK)
          return fail_be(("instruction " + std::to_string(i)).c_str());
        if (run == 0) continue;
        const double ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
        std::string key = "op" + std::to_string(program[i].opcode);
        const uint16_t op = program[i].opcode;
        if ((op >= see::kGemmNN && op <= see::kGemmAccNN) || op == see::kGemmNNQ8 || op == see::kGemmNTQ8 || op == see::kGemmNNBF16 ||
            op == see::kGemmNTBF16)
          key += " M" + std::to_string(program[i].out[0]) + " N" + std::to_string(program[i].out[1]) + " K" +
                 std::to_string(program[i].out[2]);
        rows[key].first += ms;
        ++rows[key].second;
        total += ms;
      }
    }
    std::vector<std::pair<std::string, std::pair<double, uint64_t>>> sorted(rows.begin(), rows.end());
    std::sort(sorted.begin(), sorted.end(), [](const auto& x, const auto& y) { return x.second.first > y.second.first; });
    const double n = static_cast<double>(o.profiled);
    std::printf("{\"backend\": \"%s\", \"executions\": %" PRIu64 ", \"ms_per_execution\": %.4f, "
                "\"relaxed_executions\": %" PRIu64 ", \"rows\": [",
                see_cuda_name(be), o.profiled, total / n, counters().relaxed_executions - relaxed0);
    for (size_t i = 0; i < sorted.size(); ++i)
      std::printf("%s{\"key\": \"%s\", \"ms\": %.4f, \"calls\": %" PRIu64 "}", i ? ", " : "", sorted[i].first.c_str(),
                  sorted[i].second.first / n, sorted[i].second.second / o.profiled);
    std::printf("]}\n");
  } else if (!o.trace.empty()) {
    std::vector<uint8_t> trace;
    Put<uint32_t>(&trace, 0x54504553u);   // "SEPT"
    Put<uint32_t>(&trace, 2);
    Put<uint64_t>(&trace, count);
    for (size_t i = 0; i < count; ++i) {
      const uint64_t relaxed_before = counters().relaxed_executions;
      if (see_cuda_execute(be, &program[i], &params) != SEE_OK || see_cuda_flush(be) != SEE_OK)
        return fail_be(("instruction " + std::to_string(i)).c_str());
      uint16_t writes = 0;
      for (size_t k = 0; k < extents[i].count; ++k) writes += extents[i].e[k].write ? 1 : 0;
      Put<uint32_t>(&trace, static_cast<uint32_t>(i));
      Put<uint16_t>(&trace, program[i].opcode);
      Put<uint16_t>(&trace, writes);
      Put<uint32_t>(&trace, static_cast<uint32_t>(counters().relaxed_executions - relaxed_before));
      for (size_t k = 0; k < extents[i].count; ++k) {
        const see::Extent& e = extents[i].e[k];
        if (!e.write) continue;
        Put<uint64_t>(&trace, e.off);
        Put<uint64_t>(&trace, e.bytes);
        trace.insert(trace.end(), image.begin() + static_cast<long>(e.off), image.begin() + static_cast<long>(e.off + e.bytes));
      }
    }
    if (!WriteWhole(o.trace, trace.data(), trace.size())) return fail_be("short write to the trace");
  } else {
    if (const int rc = run_all(); rc != 0) return fail_be(rc > 0 ? "execute" : "flush");
  }

  if (!WriteWhole(o.arena_out, image.data(), h.arena_size)) return fail_be("short write to the arena image");
  std::fprintf(stderr, "see-cuda-plan-probe: %s, %zu instruction(s), %s, %" PRIu64 " relaxed-kernel execution(s)\n",
               o.section.c_str(), static_cast<size_t>(count), see_cuda_name(be), counters().relaxed_executions);
  see_cuda_destroy(be);
  return 0;
}
