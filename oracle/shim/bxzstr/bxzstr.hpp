/*
 * TEST INFRASTRUCTURE - stand-in for the compressed-stream header that
 * mlx/data/core/CSVReader.h:10 and mlx/data/stream/LineReader.h:9 include.
 * Text readers are outside the transform-and-batch path; the stream passes
 * bytes through unchanged.
 */
#ifndef MLXD_ORACLE_SHIM_BXZSTR_HPP
#define MLXD_ORACLE_SHIM_BXZSTR_HPP

#include <fstream>
#include <istream>
#include <memory>
#include <sstream>
#include <string>

namespace bxz {
class istream : public std::istream {
 public:
  explicit istream(std::istream& s) : std::istream(s.rdbuf()) {}
};
} // namespace bxz

#endif
