// TEST INFRASTRUCTURE ONLY (checker, never the product path).
//
// Link glue for compiling the reference's CPU operator sources
// (fairseq/csrc/ops/{ema_hidden,ema_parameters,sequence_norm,timestep_norm}.cc)
// into a CPU-only Python extension.  Those translation units dispatch to
// *CUDAFwd / *CUDABwd symbols that live in the reference's .cu files; this
// file satisfies the linker with definitions that refuse to run, and registers
// the four op families on a pybind11 module the same way
// fairseq/csrc/mega2_extension.cc:14-24 does for the full extension.
#include "ops/ema_hidden.h"
#include "ops/ema_parameters.h"
#include "ops/sequence_norm.h"
#include "ops/timestep_norm.h"

#define MEGA_ORACLE_NO_GPU() \
  TORCH_CHECK(false, "oracle/_ref is a CPU-only build of the reference ops")

namespace mega2 {
namespace ops {

using T = torch::Tensor;
using OT = c10::optional<torch::Tensor>;

// ema_hidden.h
std::tuple<T, OT> EMAHiddenCUDAFwd(const T&, const T&, const T&, const OT&) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, OT> EMAHiddenCUDABwd(const T&, const T&, const T&, const T&,
                                         const OT&, const OT&) {
  MEGA_ORACLE_NO_GPU();
}

// ema_parameters.h
std::tuple<T, OT, OT> EMAParametersCUDAFwd(const T&, const T&, const T&,
                                           const OT&, int64_t) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, OT> EMAParametersCUDABwd(const T&, const OT&, const T&,
                                             const T&, const T&, const OT&,
                                             const OT&) {
  MEGA_ORACLE_NO_GPU();
}

// sequence_norm.h
std::tuple<T, T, T, T> SequenceNormCUDAFwd(const T&, const T&, const T&,
                                           const OT&, double, bool) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T> SequenceNormCUDABwd(const T&, const T&, const T&, const T&,
                                        const T&, const T&, const OT&, bool) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, T> GroupSequenceNormCUDAFwd(const T&, const T&, const T&,
                                                const OT&, int64_t, double,
                                                bool) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T> GroupSequenceNormCUDABwd(const T&, const T&, const T&,
                                             const T&, const T&, const T&,
                                             const OT&, int64_t, bool) {
  MEGA_ORACLE_NO_GPU();
}

// timestep_norm.h
std::tuple<T, T, T, T, T, T> TimestepNormCUDAFwd(const T&, const T&, const T&,
                                                 const T&, const T&, const T&,
                                                 const OT&, double) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, T, T> TimestepNormCUDABwd(const T&, const T&, const T&,
                                              const T&, const T&, const T&,
                                              const T&, const T&, const T&,
                                              const OT&) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, T, T, T, T> GroupTimestepNormCUDAFwd(
    const T&, const T&, const T&, const T&, const T&, const T&, const OT&,
    int64_t, double) {
  MEGA_ORACLE_NO_GPU();
}
std::tuple<T, T, T, T, T> GroupTimestepNormCUDABwd(
    const T&, const T&, const T&, const T&, const T&, const T&, const T&,
    const T&, const T&, const T&, const OT&, int64_t) {
  MEGA_ORACLE_NO_GPU();
}

}  // namespace ops

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::module m_ops = m.def_submodule("ops", "reference CPU ops");
  ops::DefineEMAHiddenOp(m_ops);
  ops::DefineEMAParametersOp(m_ops);
  ops::DefineSequenceNormOp(m_ops);
  ops::DefineTimestepNormOp(m_ops);
}

}  // namespace mega2
