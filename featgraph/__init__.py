"""Import-path shim: ``featgraph.module`` / ``featgraph.util`` / ``featgraph.op`` resolve to
featgraph_b200, so code written against dglai/FeatGraph's package imports unchanged."""
from featgraph_b200 import placeholder  # noqa: F401
