"""B200 (sm_100a) build of the ``consumer_int8`` W8A8 linear operators.

``consumer_int8.ops`` exposes the operator handles; importing it loads the prebuilt
``_C.so`` / ``libci8.so`` next to this file and never compiles anything.
"""
