"""Native kernels: build script, ctypes binding and thin functional wrappers used by tests."""
