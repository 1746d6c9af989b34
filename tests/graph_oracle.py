"""Node-by-node evaluation of a graph with the CPU oracle (kept under this name for the tests; the code lives with
the oracle)."""
from oracle.graph_eval import evaluate  # noqa: F401
