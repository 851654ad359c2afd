"""Small web front end: browse stored sessions, read a transcript, continue a conversation
(rollouts/frontend/server.py:47; the reference's terminal UI is not rebuilt, `cli.py chat` covers it).

    python -m research_b200.frontend.server --store ~/.research_b200/sessions --port 8765

Routes: ``/`` session list, ``/session/<id>`` transcript (HTML from ``agents.export``), ``/api/sessions``
and ``/api/session/<id>`` JSON, ``POST /api/session/<id>/message`` appends a user message and runs the
agent one turn with the provider stored in the session (needs that provider to be reachable).
"""

from __future__ import annotations

import argparse
import html
import time

from ..agents.export import session_to_html
from ..agents.store import FileSessionStore


def create_app(store: FileSessionStore, rollout_override=None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import HTMLResponse

    app = FastAPI(title="research_b200 sessions")

    async def load(sid: str):
        try:
            return await store.get(sid)
        except (FileNotFoundError, KeyError) as e:
            raise HTTPException(404, f"no session {sid}") from e

    @app.get("/", response_class=HTMLResponse)
    async def index():
        rows = []
        for s in sorted(await store.list(), key=lambda s: s.updated_at, reverse=True):
            when = time.strftime("%Y-%m-%d %H:%M", time.localtime(s.updated_at))
            rows.append(f"<tr><td><a href='/session/{html.escape(s.session_id)}'>{html.escape(s.session_id)}</a></td><td>{when}</td>"
                        f"<td>{html.escape(str(s.endpoint.get('provider', '?')))}/{html.escape(str(s.endpoint.get('model', '?')))}</td>"
                        f"<td>{s.num_messages}</td><td>{html.escape(s.status)}</td></tr>")
        return ("<!doctype html><meta charset='utf-8'><title>sessions</title><style>body{font-family:system-ui;margin:2rem}"
                "td,th{padding:.3rem .8rem;text-align:left}</style><h1>Sessions</h1><table><tr><th>id</th><th>updated</th>"
                "<th>model</th><th>messages</th><th>status</th></tr>" + "".join(rows) + "</table>")

    @app.get("/session/{sid}", response_class=HTMLResponse)
    async def session_page(sid: str):
        session, messages = await load(sid)
        return session_to_html(session, messages)

    @app.get("/api/sessions")
    async def api_sessions():
        return [{"id": s.session_id, "updated_at": s.updated_at, "status": s.status, "num_messages": s.num_messages,
                 "endpoint": s.endpoint, "parent_id": s.parent_id} for s in await store.list()]

    @app.get("/api/session/{sid}")
    async def api_session(sid: str):
        session, messages = await load(sid)
        return {"id": session.session_id, "status": session.status, "messages": [m.to_dict() for m in messages]}

    @app.post("/api/session/{sid}/message")
    async def api_message(sid: str, body: dict):
        from ..agents.agents import run_agent
        from ..agents.dtypes import Actor, AgentState, Endpoint, Message, RunConfig, Trajectory
        from ..agents.providers import register_provider

        session, messages = await load(sid)
        text = str(body.get("content", "")).strip()
        if not text:
            raise HTTPException(400, "content is required")
        ep = Endpoint(**{k: v for k, v in session.endpoint.items() if k in Endpoint.__dataclass_fields__})
        if rollout_override is not None:
            register_provider(ep.provider, rollout_override)
        user = Message("user", text)
        await store.append_message(sid, user)
        state = AgentState(Actor(Trajectory(tuple(messages) + (user,)), ep), None, max_turns=1, session_id=sid)
        final = (await run_agent(state, RunConfig(session_store=store)))[-1]
        reply = final.actor.trajectory.messages[-1]
        return {"role": reply.role, "content": reply.text(), "stop": final.stop.value if final.stop else None}

    return app


def main() -> None:
    import os

    import uvicorn

    ap = argparse.ArgumentParser()
    ap.add_argument("--store", default=os.path.join(os.path.expanduser("~"), ".research_b200", "sessions"))
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8765)
    args = ap.parse_args()
    uvicorn.run(create_app(FileSessionStore(args.store)), host=args.host, port=args.port, log_level="warning")


if __name__ == "__main__":
    main()
