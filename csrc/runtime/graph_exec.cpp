// The per-call walk of a built graph (flodl/src/graph/graph.rs:440-619 `forward_impl`) as a native object.
//
// `Graph.build()` hands over everything that is fixed once the graph exists: the Kahn levels, how many input ports
// each node has, where the graph's inputs go, for every node the list of (output port -> node, input port) routes,
// which outputs feed forward-reference state and which are captured under a tag, and the node to return. `forward`
// then runs the nodes level by level: it gathers a node's inputs from the value slots, fills reference ports that
// have no data yet with zeros shaped like the primary input, calls the node (a Python callable: list in, list out),
// and scatters the outputs along the precomputed routes. Values are opaque Python objects here; the only operation
// on them is `zeros_like`, supplied by the caller.
//
// Profiling (per-node wall times) stays with the Python walk: it is a debugging mode, not the hot path.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace py = pybind11;

namespace {

struct Route { int64_t from_port, to_node, to_port; };

class GraphExec {
 public:
  GraphExec(std::vector<std::vector<int64_t>> levels, std::vector<int64_t> input_count, std::vector<int64_t> port_count,
            std::vector<std::pair<int64_t, int64_t>> input_routes, std::vector<std::vector<std::tuple<int64_t, int64_t, int64_t>>> routes_from,
            std::vector<std::vector<std::pair<int64_t, int64_t>>> state_writers, std::vector<std::vector<std::pair<std::string, int64_t>>> tag_capture,
            int64_t output_node, int64_t output_port, std::vector<py::object> runs, std::vector<std::string> ids, py::object zeros_like)
      : levels_(std::move(levels)), input_count_(std::move(input_count)), port_count_(std::move(port_count)), input_routes_(std::move(input_routes)),
        state_writers_(std::move(state_writers)), tag_capture_(std::move(tag_capture)), output_node_(output_node), output_port_(output_port),
        runs_(std::move(runs)), ids_(std::move(ids)), zeros_like_(std::move(zeros_like)) {
    const size_t n = input_count_.size();
    if (port_count_.size() != n || routes_from.size() != n || state_writers_.size() != n || tag_capture_.size() != n || runs_.size() != n || ids_.size() != n)
      throw std::runtime_error("GraphExec: per-node tables differ in length");
    routes_.resize(n);
    for (size_t i = 0; i < n; ++i)
      for (const auto& r : routes_from[i]) {
        const int64_t tn = std::get<1>(r), tp = std::get<2>(r);
        if (tn < 0 || tn >= static_cast<int64_t>(n) || tp < 0) throw std::runtime_error("GraphExec: route target out of range");
        routes_[i].push_back({std::get<0>(r), tn, tp});
      }
    for (const auto& level : levels_)
      for (int64_t ni : level)
        if (ni < 0 || ni >= static_cast<int64_t>(n)) throw std::runtime_error("GraphExec: level entry out of range");
    for (const auto& ir : input_routes_)
      if (ir.first < 0 || ir.first >= static_cast<int64_t>(n) || ir.second < 0) throw std::runtime_error("GraphExec: input route out of range");
    has_tags_ = false;
    for (const auto& t : tag_capture_) has_tags_ = has_tags_ || !t.empty();
  }

  // inputs: the graph's inputs in declaration order.
  // Returns (output value, {tag: value}, [(state index, value), ...]).
  py::tuple forward(const std::vector<py::object>& inputs) const {
    if (inputs.size() != input_routes_.size())
      throw std::runtime_error("expected " + std::to_string(input_routes_.size()) + " inputs, got " + std::to_string(inputs.size()));
    const size_t n = input_count_.size();
    std::vector<std::vector<py::object>> slots(n);
    for (size_t i = 0; i < n; ++i) slots[i].assign(static_cast<size_t>(std::max<int64_t>(input_count_[i], port_count_[i])), py::none());
    for (size_t i = 0; i < inputs.size(); ++i) put(slots, input_routes_[i].first, input_routes_[i].second, inputs[i]);
    py::dict tagged;
    py::list state;
    py::object final_value = py::none();
    bool have_final = false;
    for (const auto& level : levels_) {
      for (int64_t ni : level) {
        std::vector<py::object>& ins = slots[ni];
        for (size_t p = 0; p < ins.size(); ++p) {
          if (!ins[p].is_none()) continue;
          if (p > 0) {
            if (ins[0].is_none())
              throw std::runtime_error("node '" + ids_[ni] + "': ref port " + std::to_string(p) +
                                       " has no data and primary input is also missing — check that all inputs are connected");
            ins[p] = zeros_like_(ins[0]);
          } else if (port_count_[ni] > 0) {
            throw std::runtime_error("node '" + ids_[ni] + "': missing primary input (port 0) — check that all inputs to this node are "
                                     "connected in the graph builder");
          }
        }
        py::list arg;
        for (auto& v : ins) arg.append(v);
        ins.clear();                                   // the node owns its inputs from here: free the slot's references
        py::object res = runs_[ni](arg);
        py::sequence outs = py::reinterpret_borrow<py::sequence>(res);
        const int64_t n_out = static_cast<int64_t>(py::len(outs));
        for (const Route& r : routes_[ni]) put(slots, r.to_node, r.to_port, r.from_port < n_out ? py::object(outs[r.from_port]) : py::object(py::none()));
        for (const auto& sw : state_writers_[ni])
          if (sw.second < n_out) state.append(py::make_tuple(sw.first, outs[sw.second]));
        if (has_tags_)
          for (const auto& tc : tag_capture_[ni])
            if (tc.second < n_out) tagged[py::str(tc.first)] = outs[tc.second];
        if (ni == output_node_) {
          if (output_port_ >= n_out) throw std::runtime_error("graph produced no output");
          final_value = outs[output_port_];
          have_final = true;
        }
      }
    }
    if (!have_final) throw std::runtime_error("graph produced no output");
    return py::make_tuple(final_value, tagged, state);
  }

  size_t node_count() const { return input_count_.size(); }
  size_t level_count() const { return levels_.size(); }

 private:
  static void put(std::vector<std::vector<py::object>>& slots, int64_t node, int64_t port, py::object v) {
    auto& s = slots[node];
    if (static_cast<size_t>(port) >= s.size()) s.resize(static_cast<size_t>(port) + 1, py::none());     // a port added by a late `using`
    s[port] = std::move(v);
  }

  std::vector<std::vector<int64_t>> levels_;
  std::vector<int64_t> input_count_, port_count_;
  std::vector<std::pair<int64_t, int64_t>> input_routes_;
  std::vector<std::vector<Route>> routes_;
  std::vector<std::vector<std::pair<int64_t, int64_t>>> state_writers_;
  std::vector<std::vector<std::pair<std::string, int64_t>>> tag_capture_;
  int64_t output_node_, output_port_;
  std::vector<py::object> runs_;
  std::vector<std::string> ids_;
  py::object zeros_like_;
  bool has_tags_ = false;
};

}  // namespace

void bind_graph_exec(py::module_& m) {
  py::class_<GraphExec>(m, "GraphExec")
      .def(py::init<std::vector<std::vector<int64_t>>, std::vector<int64_t>, std::vector<int64_t>, std::vector<std::pair<int64_t, int64_t>>,
                    std::vector<std::vector<std::tuple<int64_t, int64_t, int64_t>>>, std::vector<std::vector<std::pair<int64_t, int64_t>>>,
                    std::vector<std::vector<std::pair<std::string, int64_t>>>, int64_t, int64_t, std::vector<py::object>, std::vector<std::string>,
                    py::object>(),
           py::arg("levels"), py::arg("input_count"), py::arg("port_count"), py::arg("input_routes"), py::arg("routes_from"), py::arg("state_writers"),
           py::arg("tag_capture"), py::arg("output_node"), py::arg("output_port"), py::arg("runs"), py::arg("ids"), py::arg("zeros_like"))
      .def("forward", &GraphExec::forward)
      .def("node_count", &GraphExec::node_count)
      .def("level_count", &GraphExec::level_count);
}
