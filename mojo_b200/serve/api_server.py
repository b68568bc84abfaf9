"""FastAPI application over the engine.

The engine's hot loop runs in its own thread (`AsyncEngine`): HTTP handlers enqueue requests and receive tokens
through per-request asyncio queues, the engine thread drains the inbox between steps. This is the product's form of
the reference's coroutine plumbing (stdlib/src/builtin/coroutine.mojo:83-249): asyncio on the serving side, a plain
loop on the device side. A watchdog records the time of the last completed step; `/health` turns unhealthy when the
loop stops making progress while requests are pending, or when a kernel reported an error status.

Tensor-parallel serving: only rank 0 runs the HTTP application. Before every engine iteration it broadcasts the
requests it admits and aborts (`RankSync`, host-side gloo group); every rank applies the same commands in the same
order and then takes the same step, so the engines, whose kernels meet in collectives, never diverge. The other
ranks run `follower_loop` instead of a server.

Data-parallel serving (`RankSync(info, data_parallel=True)`: independent replicas, or data-parallel attention with
expert-parallel MoE) uses the same broadcast, but a request is admitted only by the rank that owns it
(request id modulo the number of ranks), every rank steps whenever any rank has work (an expert-parallel rank
without requests still joins the MoE layers), and the outputs of each iteration are gathered to rank 0, which
feeds the HTTP streams.
"""
from __future__ import annotations

import asyncio
import json
import queue
import threading
import time
import uuid

from ..engine import SamplingParams


class RankSync:
    """Command broadcast from rank 0 to the other ranks of a group, once per engine iteration; with `data_parallel`
    also the routing of requests to their owner rank and the gather of each iteration's outputs to rank 0."""

    def __init__(self, info, data_parallel: bool = False):
        self.info = info
        self.data_parallel = data_parallel

    def owns(self, rid: int) -> bool:
        return not self.data_parallel or rid % self.info.world_size == self.info.rank

    def any_failed(self, failed: bool) -> bool:
        """Whether the step that just ran failed on any rank (one small host all-reduce). Ranks that share collectives
        must take the same decision after a failure, or their next steps would not match."""
        import torch
        import torch.distributed as dist

        flag = torch.tensor([1 if failed else 0], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.info.host_group)
        return bool(flag[0])

    def gather(self, item):
        """Every rank contributes one object; rank 0 gets the list (by rank), the others None."""
        import torch.distributed as dist

        box = [None] * self.info.world_size if self.leader else None
        dist.gather_object(item, box, dst=0, group=self.info.host_group)
        return box

    @property
    def leader(self) -> bool:
        return self.info.rank == 0

    def exchange(self, cmds):
        """Rank 0 passes its command list, the others pass None; everyone gets rank 0's list."""
        from ..parallel import host_broadcast_object

        return host_broadcast_object(cmds, self.info)


def _apply(eng, cmds, on_error=None, sync: "RankSync | None" = None) -> bool:
    """Apply broadcast commands to an engine; returns False when a stop command was among them. Under data
    parallelism only the owner of a request admits or aborts it."""
    go = True
    for c in cmds:
        if c[0] in ("add", "abort") and sync is not None and not sync.owns(c[1]):
            continue
        if c[0] == "add":
            _, rid, ids, sp = c
            try:
                eng.add_request(ids, SamplingParams(**sp), request_id=rid)
            except Exception as e:  # noqa: BLE001  (bad request: every rank refuses it alike)
                if on_error is not None:
                    on_error(rid, str(e))
        elif c[0] == "abort":
            eng.abort_request(c[1])
            eng.forget(c[1])
        elif c[0] == "stop":
            go = False
    return go


def follower_loop(llm, sync: RankSync, idle_sleep: float = 0.0) -> None:
    """Ranks other than 0 of a multi-rank server: apply rank 0's commands, step when there is work."""
    eng = llm.engine
    refused: list = []
    while True:
        msg = sync.exchange(None)
        if not _apply(eng, msg["cmds"], lambda rid, err: refused.append((rid, err)), sync):
            return
        outs = []
        stepping = msg["any_busy"] if sync.data_parallel else eng.has_unfinished()
        if stepping:
            failed = False
            try:
                outs = eng.step()
            except Exception:  # noqa: BLE001  (reported to rank 0 through the flag below; this rank stays in the group)
                failed = True
            if sync.any_failed(failed):
                for rid in eng.abort_all():
                    eng.forget(rid)
                outs = []
        elif idle_sleep:
            time.sleep(idle_sleep)
        if sync.data_parallel:
            sync.gather({"outs": outs, "busy": eng.has_unfinished(), "refused": refused})
            refused = []
        for o in outs:
            if o.finished:
                eng.forget(o.request_id)


class AsyncEngine:
    def __init__(self, llm, sync: RankSync | None = None):
        self.llm = llm
        self.engine = llm.engine
        self.sync = sync
        self._any_busy = False     # data parallelism: whether any rank had unfinished requests after the last iteration
        self.inbox: queue.Queue = queue.Queue()
        self.streams: dict[int, tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self.last_step = time.time()
        self.error: str | None = None
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._loop, daemon=True, name="b2-engine")
        self.thread.start()

    def _loop(self) -> None:
        from dataclasses import asdict

        eng = self.engine
        while True:
            stopping = self._stop.is_set()
            cmds = [("stop",)] if stopping else []
            try:
                while not stopping:
                    kind, payload = self.inbox.get_nowait()
                    if kind == "add":
                        rid, ids, sp, loop, q = payload
                        self.streams[rid] = (loop, q)
                        cmds.append(("add", rid, list(ids), asdict(sp)))
                    elif kind == "abort":
                        self.streams.pop(payload, None)
                        cmds.append(("abort", payload))
            except queue.Empty:
                pass
            step_now = False
            if self.sync is not None:
                # data parallelism: every rank steps in an iteration or none does (expert-parallel ranks meet in the MoE
                # layers), so the decision is rank 0's: some rank had work after the last iteration, or work arrives now
                step_now = self._any_busy or any(c[0] == "add" for c in cmds)
                msg = self.sync.exchange({"cmds": cmds, "any_busy": step_now})      # followers now hold the same list
                cmds = msg["cmds"]

            def refuse(rid, msg):
                s = self.streams.pop(rid, None)
                if s is not None:
                    s[0].call_soon_threadsafe(s[1].put_nowait, ("error", msg))

            if not _apply(eng, cmds, refuse, self.sync):
                return
            dp = self.sync is not None and self.sync.data_parallel
            if not dp and not eng.has_unfinished():
                self.last_step = time.time()
                time.sleep(0.001 if self.sync is None else 0.003)
                continue
            stepping = (not dp) or step_now
            failed, err = False, None
            try:
                outs = eng.step() if stepping else []
            except Exception as e:  # noqa: BLE001  (kernel status error etc.): fail in-flight requests, stay alive
                failed, err, outs = True, repr(e), []
            if stepping and self.sync is not None and self.sync.any_failed(failed) and not failed:
                failed, err = True, "a step failed on another rank"
            if failed:
                # the batch's state is unknown on at least one rank: every rank drops every in-flight request
                self.error = err
                for rid, (loop, q) in list(self.streams.items()):
                    loop.call_soon_threadsafe(q.put_nowait, ("error", err))
                self.streams.clear()
                for rid in eng.abort_all():
                    eng.forget(rid)
                if not dp:
                    continue
            if dp:
                # one gather per iteration: every rank's new tokens, whether it still has work, what it refused
                parts = self.sync.gather({"outs": outs, "busy": eng.has_unfinished(), "refused": []})
                outs = [o for part in parts for o in part["outs"]]
                self._any_busy = any(part["busy"] for part in parts)
                for part in parts:
                    for rid, err in part["refused"]:
                        refuse(rid, err)
                if not self._any_busy and not outs:
                    self.last_step = time.time()
                    time.sleep(0.003)
                    continue
            self.last_step = time.time()
            for o in outs:
                s = self.streams.get(o.request_id)
                if s is None:
                    continue
                loop, q = s
                loop.call_soon_threadsafe(q.put_nowait, ("token", (o.new_token_ids, o.finished, o.finish_reason, o.logprobs)))
                if o.finished:
                    self.streams.pop(o.request_id, None)
            for o in outs:
                if o.finished:
                    eng.forget(o.request_id)     # a server runs for days: finished requests leave no state behind

    _ids = 0
    _ids_lock = threading.Lock()

    def submit(self, ids, sp: SamplingParams) -> tuple[int, asyncio.Queue]:
        self.engine.check_prompt_len(len(ids))      # ValueError -> 400 at the endpoint, before anything is queued
        with AsyncEngine._ids_lock:
            AsyncEngine._ids += 1
            rid = AsyncEngine._ids
        q: asyncio.Queue = asyncio.Queue()
        self.inbox.put(("add", (rid, list(ids), sp, asyncio.get_running_loop(), q)))
        return rid, q

    def abort(self, rid: int) -> None:
        self.inbox.put(("abort", rid))

    def healthy(self) -> bool:
        stalled = self.engine.has_unfinished() and time.time() - self.last_step > 30.0
        return self.thread.is_alive() and not stalled

    def shutdown(self) -> None:
        """Stop the engine thread; with followers, the stop command reaches them through the next broadcast."""
        self._stop.set()
        self.thread.join(timeout=10.0)


def _logprobs_from(body: dict, chat: bool) -> int | None:
    """Completions: `logprobs: k`. Chat: `logprobs: true` with optional `top_logprobs: k`. At most 20 alternatives."""
    if chat:
        if not body.get("logprobs"):
            return None
        k = int(body.get("top_logprobs") or 0)
    else:
        if body.get("logprobs") is None or body.get("logprobs") is False:
            return None
        k = int(body.get("logprobs"))
    if k < 0 or k > 20:
        raise ValueError("logprobs / top_logprobs must be between 0 and 20")
    return k


def _refuse_unsupported(body: dict) -> None:
    """OpenAI request fields this server does not implement are refused when they ask for something (HTTP 400), never
    dropped: a client that sends `n: 4` and gets one choice back has been answered wrongly."""
    for key in ("n", "best_of"):
        if body.get(key) not in (None, 1):
            raise ValueError(f"{key} other than 1 is not supported")
    for key in ("presence_penalty", "frequency_penalty", "repetition_penalty"):
        v = body.get(key)
        if v is not None and float(v) != (1.0 if key == "repetition_penalty" else 0.0):
            raise ValueError(f"{key} is not supported")
    if body.get("logit_bias"):
        raise ValueError("logit_bias is not supported")
    if body.get("echo"):
        raise ValueError("echo is not supported")
    if body.get("suffix"):
        raise ValueError("suffix is not supported")
    if body.get("tools") or body.get("functions") or body.get("response_format") not in (None, {"type": "text"}):
        raise ValueError("tools, functions and structured response formats are not supported")


def _sampling_from(body: dict, default_max: int = 16, chat: bool = False) -> SamplingParams:
    _refuse_unsupported(body)
    stop_ids = tuple(body.get("stop_token_ids") or ())
    def given(key, default):      # absent or null means the default; 0 is a value, not "unset"
        v = body.get(key)
        return default if v is None else v

    temperature = float(given("temperature", 0.0))
    top_p = float(given("top_p", 1.0))
    top_k = int(given("top_k", 0))
    max_tokens = int(given("max_completion_tokens", given("max_tokens", default_max)))
    # ranges are checked by SamplingParams itself (ValueError -> 400 at the endpoint)
    return SamplingParams(logprobs=_logprobs_from(body, chat), temperature=temperature, top_k=top_k, top_p=top_p, max_tokens=max_tokens,
                          stop_token_ids=stop_ids, ignore_eos=bool(body.get("ignore_eos", False)), seed=body.get("seed"))


def _stops_from(body: dict) -> list[str]:
    stop = body.get("stop")
    if stop is None:
        return []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or not all(isinstance(x, str) and x for x in stop):
        raise ValueError("stop must be a non-empty string or a list of non-empty strings")
    return stop


class _TextStream:
    """Turns the token stream of one request into text deltas and watches for stop strings. Text that could still
    turn out to be the beginning of a stop string is held back until the next token settles it; at a stop the text
    is cut before the stop string (which is not returned) and the request is to be aborted."""

    def __init__(self, decode, stops: list[str]):
        self.decode, self.stops = decode, stops
        self.hold = max((len(x) for x in stops), default=1) - 1
        self.ids: list[int] = []
        self.sent = 0

    def push(self, new, finished: bool) -> tuple[str, bool]:
        """(text to emit now, whether a stop string was reached)."""
        self.ids.extend(new)
        text = self.decode(self.ids)
        hits = [i for i in (text.find(x) for x in self.stops) if i >= 0]
        if hits:
            cut = max(min(hits), self.sent)
            delta, self.sent = text[self.sent:cut], cut
            return delta, True
        end = len(text) if finished else max(self.sent, len(text) - self.hold)
        delta, self.sent = text[self.sent:end], end
        return delta, False


def build_app(llm, model_name: str = "mojo_b200", sync: RankSync | None = None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI(title="mojo_b200")
    aeng = AsyncEngine(llm, sync)
    app.state.engine = aeng
    tok = llm.tokenizer

    def text_of(ids):
        t = tok.decode(ids)
        return t if t is not None else " ".join(str(i) for i in ids)

    def lp_json(ids, lps):
        """OpenAI completions layout: tokens, their log-probabilities, and per position a map of the alternatives."""
        return {"tokens": [text_of([t]) for t in ids], "token_ids": list(ids), "token_logprobs": [lp for lp, _ in lps],
                "top_logprobs": [{text_of([t]): v for t, v in top} for _, top in lps]}

    async def collect(q, rid, stops):
        """(token ids, text, finish reason) of a whole request."""
        ts = _TextStream(text_of, stops)
        parts, lps = [], []
        while True:
            kind, payload = await q.get()
            if kind == "error":
                raise HTTPException(status_code=500, detail=payload)
            new, finished, reason, lp = payload
            delta, stopped = ts.push(new, finished)
            parts.append(delta)
            lps.extend(lp or [])
            if stopped:
                aeng.abort(rid)
                return ts.ids, "".join(parts), "stop", lps
            if finished:
                return ts.ids, "".join(parts), reason, lps

    async def sse(q, rid, make_chunk, final_chunk, stops=()):
        ts = _TextStream(text_of, list(stops))
        try:
            while True:
                kind, payload = await q.get()
                if kind == "error":
                    yield f"data: {json.dumps({'error': payload})}\n\n"
                    break
                new, finished, reason, lp = payload
                delta, stopped = ts.push(new, finished)
                if stopped:
                    finished, reason = True, "stop"
                chunk = make_chunk(new, delta, reason if finished else None)
                if lp:
                    chunk["choices"][0]["logprobs"] = lp_json(new, lp)
                yield f"data: {json.dumps(chunk)}\n\n"
                if finished:
                    if final_chunk is not None:
                        yield f"data: {json.dumps(final_chunk(reason))}\n\n"
                    break
            yield "data: [DONE]\n\n"
        finally:
            aeng.abort(rid)

    @app.get("/health")
    async def health():
        ok = aeng.healthy()
        return JSONResponse({"status": "ok" if ok else "unhealthy", "last_error": aeng.error}, status_code=200 if ok else 503)

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "mojo_b200"}]}

    @app.get("/metrics")
    async def metrics():
        m = aeng.engine.metrics()
        lines = []
        for k, v in m.items():
            if isinstance(v, (int, float)) and v is not None:
                lines.append(f"# TYPE b2_{k} gauge\nb2_{k} {v}")
        eng = aeng.engine
        lines.append(f"# TYPE b2_waiting gauge\nb2_waiting {eng.scheduler.num_waiting()}")
        lines.append(f"# TYPE b2_running gauge\nb2_running {eng.scheduler.num_running()}")
        st = eng.kv.stats()
        used = st.num_pages - st.free_pages - st.cached_pages
        lines.append(f"# TYPE b2_kv_utilisation gauge\nb2_kv_utilisation {used / max(st.num_pages, 1):.6f}")
        lines.append(f"# TYPE b2_kv_cached_pages gauge\nb2_kv_cached_pages {st.cached_pages}")
        lines.append(f"# TYPE b2_requests_finished_total counter\nb2_requests_finished_total {eng.finished_requests}")
        lines.append(f"# TYPE b2_generated_tokens_total counter\nb2_generated_tokens_total {eng.generated_tokens}")
        for name, h in eng.histograms().items():
            metric = "b2_" + name.replace("_ms", "_milliseconds")
            lines.append(f"# TYPE {metric} histogram")
            running = 0
            for bound, n in zip(h["bounds"], h["counts"]):
                running += n
                lines.append(f'{metric}_bucket{{le="{bound:g}"}} {running}')
            running += h["counts"][-1]
            lines.append(f'{metric}_bucket{{le="+Inf"}} {running}')
            lines.append(f"{metric}_sum {h['sum']:.3f}")
            lines.append(f"{metric}_count {running}")
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/v1/completions")
    async def completions(body: dict):
        prompt = body.get("prompt")
        if prompt is None:
            raise HTTPException(status_code=400, detail="prompt is required")
        try:
            ids = tok.encode(prompt)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        try:
            sp = _sampling_from(body)
            stops = _stops_from(body)
            rid, q = aeng.submit(ids, sp)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        if body.get("stream"):
            def chunk(new, text, reason):
                return {"id": cid, "object": "text_completion", "created": created, "model": model_name,
                        "choices": [{"index": 0, "text": text, "token_ids": new, "finish_reason": reason}]}
            return StreamingResponse(sse(q, rid, chunk, None, stops), media_type="text/event-stream")
        out, text, reason, lps = await collect(q, rid, stops)
        return {"id": cid, "object": "text_completion", "created": created, "model": model_name,
                "choices": [{"index": 0, "text": text, "token_ids": out, "finish_reason": reason,
                             "logprobs": lp_json(out, lps) if sp.logprobs is not None else None}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}}

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        messages = body.get("messages")
        if not messages:
            raise HTTPException(status_code=400, detail="messages is required")
        ids = tok.apply_chat_template(messages)
        try:
            sp = _sampling_from(body, default_max=256, chat=True)
            stops = _stops_from(body)
            rid, q = aeng.submit(ids, sp)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        if body.get("stream"):
            first = {"sent": False}

            def chunk(new, text, reason):
                delta = {"content": text}
                if not first["sent"]:
                    delta["role"] = "assistant"
                    first["sent"] = True
                return {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                        "choices": [{"index": 0, "delta": delta, "finish_reason": reason}]}
            return StreamingResponse(sse(q, rid, chunk, None, stops), media_type="text/event-stream")
        out, text, reason, lps = await collect(q, rid, stops)
        chat_lp = None
        if sp.logprobs is not None:
            chat_lp = {"content": [{"token": text_of([t]), "logprob": lp, "top_logprobs": [{"token": text_of([a]), "logprob": v} for a, v in top]}
                                   for t, (lp, top) in zip(out, lps)]}
        return {"id": cid, "object": "chat.completion", "created": created, "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason, "logprobs": chat_lp}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}}

    return app
