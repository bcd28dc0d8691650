"""Native sm_100a kernel library: build, manifest, runtime loading and ctypes bindings."""
