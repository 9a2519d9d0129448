// Move vocabulary of the reference (utils/vocab.py:9-438), generated instead of stored:
// entries [0,1792): every (from,to) pair a queen or a knight connects, from-square major in
// a1,b1,...,h8 order; [1792,1858): white promotions (file a..h, capture-left / push / capture-right,
// pieces q r b); [1858,1924): the same for Black (rank 2 -> 1); [1924,1929): special tokens.
#pragma once
#include <cstdlib>
#include <string>
#include <vector>

namespace crl {

struct Vocab {
  std::vector<std::string> moves;      // 1929 entries
  std::vector<short> from_to;          // [1858] from*64+to, a1 = 0 ... h8 = 63
  std::vector<signed char> promo;      // [1858] 0 none, 1 q, 2 r, 3 b
  std::vector<int> mirror;             // [1858] index of the rank-mirrored move in `moves`

  static const Vocab& get() {
    static const Vocab v = build();
    return v;
  }

 private:
  static std::string sq(int s) {
    std::string r;
    r += static_cast<char>('a' + (s & 7));
    r += static_cast<char>('1' + (s >> 3));
    return r;
  }
  static void promotions(std::vector<std::string>& out, char from_rank, char to_rank) {
    static const char pieces[3] = {'q', 'r', 'b'};
    for (int f = 0; f < 8; ++f)
      for (int tf = f - 1; tf <= f + 1; ++tf) {
        if (tf < 0 || tf > 7) continue;
        for (char pc : pieces) {
          std::string m;
          m += static_cast<char>('a' + f); m += from_rank;
          m += static_cast<char>('a' + tf); m += to_rank;
          m += pc;
          out.push_back(m);
        }
      }
  }
  static Vocab build() {
    Vocab v;
    for (int a = 0; a < 64; ++a)
      for (int b = 0; b < 64; ++b) {
        if (a == b) continue;
        const int df = std::abs((a & 7) - (b & 7)), dr = std::abs((a >> 3) - (b >> 3));
        if (df == 0 || dr == 0 || df == dr || (df == 1 && dr == 2) || (df == 2 && dr == 1))
          v.moves.push_back(sq(a) + sq(b));
      }
    promotions(v.moves, '7', '8');
    const size_t n_leela = v.moves.size();
    promotions(v.moves, '2', '1');
    for (const char* t : {"<thinking>", "</thinking>", "end_variation", "end", "padding_token"})
      v.moves.push_back(t);
    for (size_t i = 0; i < n_leela; ++i) {
      const std::string& m = v.moves[i];
      const int from = (m[0] - 'a') + 8 * (m[1] - '1'), to = (m[2] - 'a') + 8 * (m[3] - '1');
      v.from_to.push_back(static_cast<short>(from * 64 + to));
      signed char p = 0;
      if (m.size() == 5) p = m[4] == 'q' ? 1 : (m[4] == 'r' ? 2 : 3);
      v.promo.push_back(p);
      std::string mir = m;
      mir[1] = static_cast<char>('1' + ('8' - m[1]));
      mir[3] = static_cast<char>('1' + ('8' - m[3]));
      int found = -1;
      for (size_t j = 0; j < v.moves.size(); ++j)
        if (v.moves[j] == mir) { found = static_cast<int>(j); break; }
      v.mirror.push_back(found);
    }
    return v;
  }
};

}  // namespace crl
