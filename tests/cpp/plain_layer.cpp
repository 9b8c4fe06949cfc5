// Runs the float64 transformer layer of oracle/transformer_plain.h on data
// from a file, so that a Python test can compare it with an independent
// implementation (host only, no GPU).
//
//   plain_layer <in.bin> <out.bin>
// in.bin: int32 seq_len, hidden, heads, ffn, exact, degrees[4] (exp, inv, rsqrt, gelu);
//         float64 score_range, sum_lo, sum_hi, var_lo, var_hi, gelu_range, ln_eps;
//         float64 arrays: the four coefficient vectors, wq wk wv wo w1 w2 bq bk bv bo b1 b2
//         gamma1 beta1 gamma2 beta2, x[seq_len][hidden].
// out.bin: float64 out[seq_len][hidden].
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <algorithm>
#include <iostream>
#include <string>

#include "../../oracle/transformer_plain.h"
#include "cheddar/RankGroup.h"

// plain_layer --blocks: checks the block partition the sharded layer uses
// (every item owned exactly once, sizes differ by at most one, owner lookup
// consistent) for the shapes that occur; prints "blocks ok".
static int CheckBlocks() {
  for (int n : {1, 2, 12, 32, 64, 768, 3072})
    for (int world = 1; world <= 8; world++) {
      int next = 0, smallest = n, largest = 0;
      for (int r = 0; r < world; r++) {
        const auto [lo, hi] = cheddar::BlockOfRank(n, world, r);
        if (lo != next || hi < lo) return 1;
        for (int i = lo; i < hi; i++)
          if (cheddar::RankOfItem(n, world, i) != r) return 1;
        smallest = std::min(smallest, hi - lo);
        largest = std::max(largest, hi - lo);
        next = hi;
      }
      if (next != n || largest - smallest > 1) return 1;
    }
  std::cout << "blocks ok" << std::endl;
  return 0;
}

int main(int argc, char **argv) {
  if (argc == 2 && std::string(argv[1]) == "--blocks") return CheckBlocks();
  if (argc < 3) return 2;
  std::ifstream in(argv[1], std::ios::binary);
  int32_t head[9];
  in.read(reinterpret_cast<char *>(head), sizeof(head));
  double par[7];
  in.read(reinterpret_cast<char *>(par), sizeof(par));
  const int T = head[0], H = head[1], heads = head[2], F = head[3];
  auto vec = [&](size_t n) {
    std::vector<double> v(n);
    in.read(reinterpret_cast<char *>(v.data()), (std::streamsize)(n * sizeof(double)));
    return v;
  };
  plain_transformer::Spec s{T, H, heads, H / heads, F, par[0], par[1], par[2], par[3], par[4], par[5], par[6],
                            vec(head[5] + 1), vec(head[6] + 1), vec(head[7] + 1), vec(head[8] + 1), head[4] != 0};
  auto wq = vec((size_t)H * H), wk = vec((size_t)H * H), wv = vec((size_t)H * H), wo = vec((size_t)H * H);
  auto w1 = vec((size_t)H * F), w2 = vec((size_t)F * H);
  auto bq = vec(H), bk = vec(H), bv = vec(H), bo = vec(H), b1 = vec(F), b2 = vec(H);
  auto g1 = vec(H), be1 = vec(H), g2 = vec(H), be2 = vec(H);
  auto x = vec((size_t)T * H);
  if (!in) {
    std::cerr << "plain_layer: short input\n";
    return 1;
  }
  plain_transformer::Weights w{wq.data(), wk.data(), wv.data(), wo.data(), w1.data(), w2.data(), bq.data(), bk.data(),
                               bv.data(), bo.data(), b1.data(), b2.data(), g1.data(), be1.data(), g2.data(),
                               be2.data()};
  std::vector<double> out;
  plain_transformer::Layer(out, x, s, w);
  std::ofstream o(argv[2], std::ios::binary);
  o.write(reinterpret_cast<const char *>(out.data()), (std::streamsize)(out.size() * sizeof(double)));
  return 0;
}
