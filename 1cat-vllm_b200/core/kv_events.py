"""Publisher of KV-cache block events for external routers and cache-aware load balancers
(reference: vllm/distributed/kv_events.py — ``KVEventBatch`` of ``BlockStored`` / ``BlockRemoved`` / ``AllBlocksCleared`` over a ZMQ
PUB socket, msgpack-encoded, with a monotonically increasing sequence number).

Wire format: multipart ``[topic, seq (8 bytes, big endian), payload]`` where payload is msgpack
``{"ts": float, "events": [{"type": "BlockStored" | "BlockRemoved" | "AllBlocksCleared", "block_id": int, "block_hash": hex | None}, ...]}``."""
from __future__ import annotations

import time
from typing import Optional


class KVEventPublisher:
    def __init__(self, endpoint: str = "tcp://127.0.0.1:5557", topic: str = "kv-events") -> None:
        import zmq
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.PUB)
        if not endpoint.startswith("connect:"):
            self.sock.bind(endpoint)
        else:
            self.sock.connect(endpoint[len("connect:"):])  # "connect:tcp://host:port" joins a collector that binds
        self.topic = topic.encode()
        self.seq = 0

    def publish(self, events: list) -> None:
        """``events``: ``(kind, block_id, block_hash | None)`` tuples as collected by the block pool."""
        if not events:
            return
        import msgpack
        names = {"stored": "BlockStored", "removed": "BlockRemoved", "cleared": "AllBlocksCleared"}
        body = {"ts": time.time(), "events": [{"type": names.get(e[0], e[0]), "block_id": e[1], "block_hash": e[2].hex() if len(e) > 2 and e[2] else None}
                                              for e in events]}
        self.sock.send_multipart([self.topic, self.seq.to_bytes(8, "big"), msgpack.packb(body)])
        self.seq += 1

    def close(self) -> None:
        self.sock.close(linger=0)


def make_publisher(cfg: Optional[dict]) -> Optional[KVEventPublisher]:
    if not cfg or not cfg.get("enable_kv_cache_events", True):
        return None
    return KVEventPublisher(cfg.get("endpoint", "tcp://127.0.0.1:5557"), cfg.get("topic", "kv-events"))
