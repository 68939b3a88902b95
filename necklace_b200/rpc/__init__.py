"""OneRPC control plane on ZeroMQ (pyzmq + msgpack)."""
