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


def compute_talker_prompt_ids_length(thinker_input_ids: list[int], thinker_output_len: int,
                                     im_start_id: int = 151644, system_id: int = 8948) -> int:
    """Length of the talker prompt for a thinker sequence: the talker consumes the assistant
    turn (everything after the last ``<|im_start|>``) plus the generated tokens, with system
    turns dropped (adapter.py:176)."""
    starts = [i for i, t in enumerate(thinker_input_ids) if t == im_start_id]
    keep = 0
    for j, s in enumerate(starts):
        e = starts[j + 1] if j + 1 < len(starts) else len(thinker_input_ids)
        if s + 1 < len(thinker_input_ids) and thinker_input_ids[s + 1] == system_id:
            continue
        keep += e - s
    if not starts:
        keep = len(thinker_input_ids)
    return keep + thinker_output_len
