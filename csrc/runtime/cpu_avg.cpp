// Host-side parameter averaging of the asynchronous trainer's CPU backend (flodl/src/distributed/coordinator/cpu_avg.rs:540-599
// averages, :600-660 measures how far every replica was from the mean), as one pass over memory.
//
// The coordinator holds one snapshot per rank: a list of CPU tensors in the same order and shapes. The mean is weighted
// (by the batches a rank contributed); the divergence report wants, per rank, ||p_r - mean||^2 and ||p_r||^2, and
// ||mean||^2. Done with tensor operations that is 2W+1 reads and W writes of a parameter-sized temporary for the mean and
// another 3W float64 temporaries for the norms; here every element of every snapshot is read once, the mean is written
// once and the five sums ride along in registers.
//
// The sums are accumulated in double per fixed block of 16384 elements and the blocks are added in index order, so the
// result does not depend on how many threads ran (as many as ATen's intra-op setting, `torch.set_num_threads`).
#include <ATen/Parallel.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <tuple>
#include <vector>

namespace py = pybind11;
using torch::Tensor;

namespace {

constexpr int64_t kBlock = 16384;

struct Sums {
  std::vector<double> delta_sq, pre_sq;   // per rank
  double post_sq = 0.0;
};

// The two inner loops, compiled a second time for AVX2 hosts and picked when the library loads. Eight independent partial
// sums per quantity keep the double-precision additions off one dependency chain and let the compiler use vector lanes
// (it may not reassociate a single floating-point sum by itself).
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define FB_CLONES __attribute__((target_clones("avx2,fma", "default")))
#else
#define FB_CLONES
#endif

FB_CLONES void block_mean(const float* const* src, const float* w, int64_t ranks, float* out, int64_t lo, int64_t hi) {
  const float* s0 = src[0];
  const float w0 = w[0];
  for (int64_t j = lo; j < hi; ++j) out[j] = s0[j] * w0;
  for (int64_t r = 1; r < ranks; ++r) {                   // the block (64 KB) stays in cache between the passes
    const float* sr = src[r];
    const float wr = w[r];
    for (int64_t j = lo; j < hi; ++j) out[j] += wr * sr[j];
  }
}

FB_CLONES double block_sq(const float* a, int64_t lo, int64_t hi) {
  double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t j = lo;
  for (; j + 8 <= hi; j += 8)
    for (int k = 0; k < 8; ++k) {
      const double v = a[j + k];
      acc[k] += v * v;
    }
  for (; j < hi; ++j) acc[0] += static_cast<double>(a[j]) * a[j];
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

// sum (a - m)^2 and sum a^2 over [lo, hi)
FB_CLONES void block_delta_sq(const float* a, const float* m, int64_t lo, int64_t hi, double* delta_sq, double* pre_sq) {
  double d[8] = {0, 0, 0, 0, 0, 0, 0, 0}, p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t j = lo;
  for (; j + 8 <= hi; j += 8)
    for (int k = 0; k < 8; ++k) {
      const double v = a[j + k], e = v - static_cast<double>(m[j + k]);
      d[k] += e * e;
      p[k] += v * v;
    }
  for (; j < hi; ++j) {
    const double v = a[j], e = v - static_cast<double>(m[j]);
    d[0] += e * e;
    p[0] += v * v;
  }
  *delta_sq = ((d[0] + d[1]) + (d[2] + d[3])) + ((d[4] + d[5]) + (d[6] + d[7]));
  *pre_sq = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
}

// One tensor position whose replicas are all float32 and contiguous.
struct Job {
  std::vector<const float*> src;
  float* out;
  int64_t n, first_block;          // first_block: index of this tensor's first block among all jobs' blocks
};

// All jobs' blocks, handed out eight at a time to `threads` host threads (std::thread: the extension is not built with
// OpenMP, so ATen's header-only parallel_for would run serially here).
void run_jobs(const std::vector<Job>& jobs, const std::vector<float>& w, bool norms, int64_t total_blocks, int threads, Sums& sums) {
  const int64_t ranks = static_cast<int64_t>(w.size()), width = 2 * ranks + 1;
  std::vector<double> part(norms ? static_cast<size_t>(total_blocks * width) : 0, 0.0);
  std::atomic<int64_t> next{0};
  constexpr int64_t kGrab = 8;
  auto work = [&] {
    size_t ji = 0;
    for (;;) {
      const int64_t g0 = next.fetch_add(kGrab, std::memory_order_relaxed);
      if (g0 >= total_blocks) return;
      const int64_t g1 = std::min(total_blocks, g0 + kGrab);
      for (int64_t g = g0; g < g1; ++g) {
        while (ji + 1 < jobs.size() && jobs[ji + 1].first_block <= g) ++ji;      // blocks only move forward for one thread
        const Job& job = jobs[ji];
        const int64_t lo = (g - job.first_block) * kBlock, hi = std::min(job.n, lo + kBlock);
        block_mean(job.src.data(), w.data(), ranks, job.out, lo, hi);
        if (!norms) continue;
        double* row = &part[static_cast<size_t>(g * width)];
        for (int64_t r = 0; r < ranks; ++r) block_delta_sq(job.src[r], job.out, lo, hi, &row[r], &row[ranks + r]);
        row[2 * ranks] = block_sq(job.out, lo, hi);
      }
    }
  };
  threads = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(threads, (total_blocks + kGrab - 1) / kGrab)));
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  if (!norms) return;
  for (int64_t g = 0; g < total_blocks; ++g) {                                   // in index order: the same sums for any thread count
    const double* row = &part[static_cast<size_t>(g * width)];
    for (int64_t r = 0; r < ranks; ++r) { sums.delta_sq[r] += row[r]; sums.pre_sq[r] += row[ranks + r]; }
    sums.post_sq += row[2 * ranks];
  }
}

// Any other floating dtype or layout: the same arithmetic through tensor operations (float32 mean, float64 norms).
Tensor average_generic(const std::vector<Tensor>& src, const std::vector<float>& w, bool norms, Sums& sums) {
  Tensor acc = src[0].to(torch::kFloat32) * w[0];
  for (size_t r = 1; r < src.size(); ++r) acc.add_(src[r].to(torch::kFloat32), w[r]);
  Tensor out = acc.to(src[0].scalar_type());
  if (norms) {
    Tensor m = out.to(torch::kFloat64);
    sums.post_sq += m.pow(2).sum().item<double>();
    for (size_t r = 0; r < src.size(); ++r) {
      Tensor v = src[r].to(torch::kFloat64);
      sums.delta_sq[r] += (v - m).pow(2).sum().item<double>();
      sums.pre_sq[r] += v.pow(2).sum().item<double>();
    }
  }
  return out;
}

// per_rank[r][i]: tensor i of rank r. weights[r]: share of rank r (they should sum to one).
// Returns (mean tensors, sum_i ||p_r,i - mean_i||^2 per rank, sum_i ||p_r,i||^2 per rank, sum_i ||mean_i||^2).
std::tuple<std::vector<Tensor>, std::vector<double>, std::vector<double>, double> cpu_weighted_average(
    const std::vector<std::vector<Tensor>>& per_rank, const std::vector<double>& weights, bool norms) {
  TORCH_CHECK(!per_rank.empty(), "cpu_weighted_average: no snapshots");
  TORCH_CHECK(weights.size() == per_rank.size(), "cpu_weighted_average: ", per_rank.size(), " snapshots but ", weights.size(), " weights");
  const size_t ranks = per_rank.size(), count = per_rank[0].size();
  for (size_t r = 1; r < ranks; ++r)
    TORCH_CHECK(per_rank[r].size() == count, "cpu_weighted_average: rank ", r, " sent ", per_rank[r].size(), " tensors, rank 0 sent ", count);
  std::vector<float> w(weights.begin(), weights.end());
  Sums sums;
  sums.delta_sq.assign(ranks, 0.0);
  sums.pre_sq.assign(ranks, 0.0);
  std::vector<Tensor> out;
  out.reserve(count);
  py::gil_scoped_release release;                          // tens of milliseconds for a large model: let the coordinator's loop run
  std::vector<Job> jobs;
  int64_t total_blocks = 0;
  for (size_t i = 0; i < count; ++i) {
    std::vector<Tensor> src(ranks);
    bool fast = true;
    for (size_t r = 0; r < ranks; ++r) {
      src[r] = per_rank[r][i].detach();
      TORCH_CHECK(!src[r].is_cuda(), "cpu_weighted_average: tensor ", i, " of rank ", r, " is not on the host");
      TORCH_CHECK(src[r].sizes() == per_rank[0][i].sizes(), "cpu_weighted_average: tensor ", i, " of rank ", r, " has shape ", src[r].sizes(),
                  ", rank 0 has ", per_rank[0][i].sizes());
      fast = fast && src[r].scalar_type() == torch::kFloat32 && src[r].is_contiguous();
    }
    if (!fast) {
      out.push_back(average_generic(src, w, norms, sums));
      continue;
    }
    Tensor mean = torch::empty_like(src[0]);
    if (mean.numel() > 0) {
      Job job;
      for (size_t r = 0; r < ranks; ++r) job.src.push_back(src[r].data_ptr<float>());     // per_rank keeps the storage alive
      job.out = mean.data_ptr<float>();
      job.n = mean.numel();
      job.first_block = total_blocks;
      total_blocks += (job.n + kBlock - 1) / kBlock;
      jobs.push_back(std::move(job));
    }
    out.push_back(std::move(mean));
  }
  if (!jobs.empty()) run_jobs(jobs, w, norms, total_blocks, at::get_num_threads(), sums);
  return {std::move(out), std::move(sums.delta_sq), std::move(sums.pre_sq), sums.post_sq};
}

}  // namespace

void bind_cpu_avg(py::module_& m) {
  m.def("cpu_weighted_average", &cpu_weighted_average, py::arg("per_rank"), py::arg("weights"), py::arg("norms") = true,
        "Weighted mean of per-rank tensor lists on the host, with the squared norms of the divergence report from the same pass.");
}
