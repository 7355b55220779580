"""torkit3d_b200: the torkit3d neighbour-search / sampling operators, hand-written for B200 (sm_100a).

``torkit3d_b200.ops`` mirrors ``torkit3d.ops``; ``torkit3d_b200._C`` mirrors the reference's
extension module and sits on the C ABI of ``libtk3d_b200.so`` (``include/tk3d.h``).
"""
__version__ = "0.1.0"
