// Graph optimizer infrastructure: a small expression-pattern matcher plus the
// pass table.  Passes are grouped in the reference's levels
// (onnxruntime/core/optimizer/graph_transformer_utils.cc:210-544): level 1 =
// basic (semantics-preserving clean-ups, constant folding, Gelu / LayerNorm
// fusion), level 2 = extended (transformer fusions into com.microsoft ops) and
// a GPU-only group that lowers GEMM chains onto the fused sm_100a kernels.
#pragma once
#include <functional>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "graph.h"
#include "session.h"

namespace ortb {
namespace opt {

// ------------------------------------------------------------- pattern DSL
struct Pat {
  enum Kind { VAR, CONST, ANYCONST, OP } kind = VAR;
  std::string name;          // VAR / ANYCONST binding name, or OP binding name (optional)
  std::string op, domain;    // OP
  double cval = 0;           // CONST
  double tol = 2e-3;         // relative tolerance for CONST
  std::vector<Pat> args;     // OP operands (positional; extra node inputs must be absent)
  bool commutative = false;  // try both operand orders (binary ops)
  bool allow_extra_inputs = false;
};

Pat V(const std::string& name);
Pat C(double value);
Pat K(const std::string& name);  // any constant initializer, bound under `name`
Pat Op(const std::string& op, std::vector<Pat> args, const std::string& bind = "");
Pat OpD(const std::string& domain, const std::string& op, std::vector<Pat> args, const std::string& bind = "");

struct Match {
  std::map<std::string, std::string> values;  // binding name -> graph value name
  std::map<std::string, Node*> nodes;         // OP binding name -> node
  std::vector<Node*> matched;                 // every node covered by the pattern, root first
};

// Match the expression rooted at the node producing `value`.  Cast nodes are looked through when
// `through_casts` is set (they are recorded in `matched`).
bool MatchExpr(const Graph& g, const std::string& value, const Pat& p, Match* m, bool through_casts = false);
// True when no interior value of the match is read outside of it (the root's outputs may be).
bool IsClosed(const Graph& g, const Match& m, const Node* root, const std::set<std::string>& allowed_escapes = {});

// scalar constant helpers
bool ScalarConst(const Graph& g, const std::string& value, double* out);
bool IsConst1D(const Graph& g, const std::string& value, int64_t* len = nullptr);

struct PassContext {
  Graph& g;
  bool gpu;
  const ConfigOptions& config;
  int world_size;
};

struct Pass {
  std::string name;
  int level;      // 1 basic, 2 extended
  bool gpu_only;
  std::function<int(PassContext&)> run;  // returns the number of rewrites
};

const std::vector<Pass>& AllPasses();

// pass groups, each in its own translation unit
void AddBasicPasses(std::vector<Pass>& v);
void AddFusionPasses(std::vector<Pass>& v);
void AddGpuPasses(std::vector<Pass>& v);
void AddMorePasses(std::vector<Pass>& v);
void AddQdqPasses(std::vector<Pass>& v);
void AddMorePasses2(std::vector<Pass>& v);
void AddMorePasses3(std::vector<Pass>& v);
void AddQdqPrepPasses(std::vector<Pass>& v);

// Replace the nodes of `m` by `fused` (already added to the graph); rewires nothing else.
void RemoveMatched(Graph& g, const Match& m);

}  // namespace opt
}  // namespace ortb
