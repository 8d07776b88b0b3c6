// schema.cpp -- op_name / op_arity tables expanded from ops.def.
#include "ad/core/schema.hpp"

namespace ag {

namespace {
struct OpInfo {
    const char* name;
    int arity;
};
constexpr OpInfo kOps[] = {
#define OP(name, arity, str) {str, arity},
#include "ad/detail/ops.def"
#undef OP
};
static_assert(sizeof(kOps) / sizeof(kOps[0]) == OpCount, "ops.def and enum Op out of step");
}  // namespace

const char* op_name(Op o) {
    const auto i = static_cast<std::size_t>(o);
    return i < OpCount ? kOps[i].name : "invalid";
}
int op_arity(Op o) {
    const auto i = static_cast<std::size_t>(o);
    return i < OpCount ? kOps[i].arity : -1;
}

}  // namespace ag
