from featgraph_b200.op import *  # noqa: F401,F403
