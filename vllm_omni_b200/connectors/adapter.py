"""Orchestrator-side use of a connector for one pipeline edge
(vllm_omni/distributed/omni_connectors/adapter.py:18-206): the payload goes into the
connector, the stage queue carries only the descriptor, and the receiving stage pulls the
payload before it schedules the request.  Transfer timings feed the metrics aggregator."""
from __future__ import annotations

import time
from typing import Any


def try_send_via_connector(connector, from_stage: int, to_stage: int, request_id: str, engine_inputs: Any,
                           task: dict, metrics=None) -> bool:
    t0 = time.perf_counter()
    ok, size, meta = connector.put(from_stage, to_stage, request_id, engine_inputs)
    tx_ms = (time.perf_counter() - t0) * 1e3
    if not ok:
        return False
    task["connector_meta"] = {"from_stage": from_stage, "to_stage": to_stage, "key": request_id, "meta": meta,
                              "size": size, "put_ts": time.time()}
    if metrics is not None:
        metrics.record_transfer_tx(from_stage, to_stage, request_id, size, tx_ms,
                                   used_shm=bool(meta and "shm" in meta),
                                   device_direct=bool(getattr(connector, "supports_device_tensors", False)))
    return True


def try_recv_via_connector(connector, task: dict, metrics=None):
    """Resolve ``task['engine_inputs']`` from its connector descriptor (no-op when inline)."""
    cm = task.get("connector_meta")
    if cm is None:
        return task.get("engine_inputs")
    t0 = time.perf_counter()
    res = connector.get(cm["from_stage"], cm["to_stage"], cm["key"], cm["meta"])
    if res is None:
        raise TimeoutError(f"payload {cm['key']} for edge {cm['from_stage']}->{cm['to_stage']} never arrived")
    data, size = res
    rx_ms = (time.perf_counter() - t0) * 1e3
    task["engine_inputs"] = data
    task["rx_stats"] = {"rx_transfer_bytes": size, "rx_decode_time_ms": rx_ms,
                        "rx_in_flight_time_ms": max(0.0, (time.time() - cm["put_ts"]) * 1e3 - rx_ms)}
    if metrics is not None:
        metrics.record_transfer_rx(cm["from_stage"], cm["to_stage"], cm["key"], rx_ms,
                                   task["rx_stats"]["rx_in_flight_time_ms"])
    return data


def compute_talker_prompt_ids_length(prompt_ids: list[int], im_start_id: int = 151644, system_id: int = 8948,
                                     user_id: int = 872, assistant_id: int = 77091) -> int:
    """Length of the talker prompt built from a thinker sequence (adapter.py:176-206): the sequence is
    cut at every ``<|im_start|>``; system turns are dropped, every user turn contributes its tokens,
    and the last assistant turn contributes nine rows (3 header tokens, 4 x tts-pad, tts-bos, the
    first reply token).  Earlier assistant turns are dropped."""
    starts = [i for i, t in enumerate(prompt_ids) if t == im_start_id] + [len(prompt_ids)]
    user_len = assistant_len = 0
    for j in range(len(starts) - 1):
        s, e = starts[j], starts[j + 1]
        role = prompt_ids[s + 1] if s + 1 < len(prompt_ids) else None
        if role == system_id:
            continue
        if role == user_id:
            user_len += e - s
        elif role == assistant_id and j == len(starts) - 2:
            assistant_len += 9
    return user_len + assistant_len
