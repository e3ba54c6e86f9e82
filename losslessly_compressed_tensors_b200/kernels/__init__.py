"""Launch layer: ctypes bindings of ``liblct_b200.so`` and one wrapper per kernel."""
