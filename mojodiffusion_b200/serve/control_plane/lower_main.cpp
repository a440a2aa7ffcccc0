// mdb-lower: reads one generation request (JSON) from stdin or a file, lowers its workflow graph and prints the flat
// request. Exit code 0 on success; on a lowering error prints {"error": ..., "status": 501|422} and exits 3.
// ``mdb-lower --node-types`` prints the node type ids the graph executor accepts (a JSON array) and exits.
#include <fstream>
#include <iostream>
#include <sstream>

#include "graph.hpp"

int main(int argc, char** argv) {
  std::stringstream ss;
  if (argc > 1 && std::string(argv[1]) == "--node-types") {
    mdb::Json arr = mdb::Json::array();
    for (auto& kv : mdb::graph::Engine::registry()) arr.push(mdb::Json(kv.first));
    std::cout << arr.dump() << "\n";
    return 0;
  }
  if (argc > 1) {
    std::ifstream f(argv[1]);
    if (!f) { std::cerr << "cannot open " << argv[1] << "\n"; return 2; }
    ss << f.rdbuf();
  } else {
    ss << std::cin.rdbuf();
  }
  mdb::Json req;
  std::string err;
  if (!mdb::Json::try_parse(ss.str(), &req, &err)) {
    mdb::Json e = mdb::Json::object();
    e.set("error", mdb::Json(err));
    e.set("status", mdb::Json(400));
    std::cout << e.dump() << "\n";
    return 3;
  }
  try {
    mdb::graph::lower_request(req);
  } catch (const mdb::graph::GraphError& ge) {
    mdb::Json e = mdb::Json::object();
    e.set("error", mdb::Json(ge.text()));
    e.set("status", mdb::Json(ge.status));
    if (ge.node_id >= 0) e.set("node_id", mdb::Json(static_cast<int64_t>(ge.node_id)));
    if (!ge.type_id.empty()) e.set("type_id", mdb::Json(ge.type_id));
    std::cout << e.dump() << "\n";
    return 3;
  }
  std::cout << req.dump() << "\n";
  return 0;
}
