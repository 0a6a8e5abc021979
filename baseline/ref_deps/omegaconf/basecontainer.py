import sys

BaseContainer = sys.modules["_ref_deps_conf"].Node
