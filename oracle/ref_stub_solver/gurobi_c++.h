/* Stand-in for the commercial solver's C++ header, which is not installed here: just enough
 * declarations (our own, with empty bodies) for the reference's solver source to COMPILE, so that
 * the placement heuristics that live in the same file (Intuitive, Rep, CliquePart: plain loops,
 * no solver involved) can be run for the parity pin under oracle/_ref/.  Anything that would
 * call the real solver does nothing here and is never used by the pin.  Test infrastructure. */
#pragma once
#include <string>

enum {
  GRB_IntParam_Method, GRB_IntParam_Presolve, GRB_IntParam_Threads, GRB_IntParam_DegenMoves,
  GRB_IntParam_ConcurrentMIP, GRB_IntParam_ScaleFlag, GRB_IntParam_PrePasses, GRB_IntParam_NormAdjust,
  GRB_IntParam_Cuts, GRB_IntParam_AggFill, GRB_IntParam_MIPFocus, GRB_IntParam_StrongCGCuts,
  GRB_IntParam_SimplexPricing, GRB_IntParam_MIRCuts, GRB_IntParam_LogToConsole, GRB_IntParam_GomoryPasses,
  GRB_IntParam_FlowCoverCuts, GRB_IntParam_CutPasses, GRB_IntParam_BranchDir, GRB_IntParam_Aggregate,
  GRB_IntParam_NodeMethod, GRB_IntParam_Crossover, GRB_IntParam_OutputFlag, GRB_IntParam_Seed,
  GRB_IntParam_VarBranch, GRB_IntParam_Symmetry, GRB_IntParam_Disconnected, GRB_IntParam_NumericFocus,
  GRB_IntParam_BarOrder, GRB_IntParam_BarHomogeneous, GRB_IntParam_Sifting, GRB_IntParam_SubMIPNodes
};
enum {
  GRB_DoubleParam_MIPGap = 1000, GRB_DoubleParam_OptimalityTol, GRB_DoubleParam_BarConvTol,
  GRB_DoubleParam_Heuristics, GRB_DoubleParam_TimeLimit, GRB_DoubleParam_NoRelHeurTime,
  GRB_DoubleParam_FeasibilityTol, GRB_DoubleParam_IntFeasTol, GRB_DoubleParam_MIPGapAbs
};
enum GRB_DoubleAttr { GRB_DoubleAttr_X = 2000, GRB_DoubleAttr_ObjVal, GRB_DoubleAttr_Runtime, GRB_DoubleAttr_MIPGap };
enum { GRB_IntAttr_Status = 3000, GRB_IntAttr_SolCount };
enum { GRB_MINIMIZE = 1, GRB_MAXIMIZE = -1 };
constexpr char GRB_CONTINUOUS = 'C';
constexpr char GRB_BINARY = 'B';
constexpr char GRB_INTEGER = 'I';

class GRBVar {
  void* p = nullptr;

 public:
  double get(int) const { return 0.0; }
  template <typename A, typename B>
  void set(A, B) {}
};

class GRBLinExpr {
 public:
  GRBLinExpr(double = 0.0) {}
  GRBLinExpr(const GRBVar&, double = 1.0) {}
  GRBLinExpr& operator+=(const GRBLinExpr&) { return *this; }
  GRBLinExpr& operator-=(const GRBLinExpr&) { return *this; }
  GRBLinExpr& operator*=(double) { return *this; }
  double getValue() const { return 0.0; }
};
inline GRBLinExpr operator+(const GRBLinExpr& a, const GRBLinExpr&) { return a; }
inline GRBLinExpr operator-(const GRBLinExpr& a, const GRBLinExpr&) { return a; }
inline GRBLinExpr operator-(const GRBLinExpr& a) { return a; }
inline GRBLinExpr operator*(double, const GRBLinExpr& a) { return a; }
inline GRBLinExpr operator*(const GRBLinExpr& a, double) { return a; }
inline GRBLinExpr operator/(const GRBLinExpr& a, double) { return a; }

class GRBTempConstr {};
inline GRBTempConstr operator<=(const GRBLinExpr&, const GRBLinExpr&) { return {}; }
inline GRBTempConstr operator>=(const GRBLinExpr&, const GRBLinExpr&) { return {}; }
inline GRBTempConstr operator==(const GRBLinExpr&, const GRBLinExpr&) { return {}; }

class GRBConstr {};

class GRBEnv {
 public:
  GRBEnv(bool = false) {}
  template <typename A, typename B>
  void set(A, B) {}
  void start() {}
};

class GRBModel {
 public:
  GRBModel(const GRBEnv&) {}
  GRBVar addVar(double, double, double, char, const std::string& = "") { return GRBVar(); }
  template <typename... A>
  GRBConstr addConstr(A&&...) { return {}; }
  template <typename... A>
  void setObjective(A&&...) {}
  template <typename A, typename B>
  void set(A, B) {}
  double get(int) const { return 0.0; }
  void optimize() {}
  void update() {}
  void reset(int = 0) {}
  void write(const std::string&) {}
};

class GRBException {
 public:
  int getErrorCode() const { return 0; }
  std::string getMessage() const { return std::string(); }
};
