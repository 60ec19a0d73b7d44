"""B200 (sm_100a) forward backend for Msnhnet nets: native libraries + thin ctypes bindings."""
