"""Small web front end: browse stored sessions, read a transcript, continue a conversation
(rollouts/frontend/server.py:47; the reference's terminal UI is not rebuilt, `cli.py chat` covers it).

    python -m research_b200.frontend.server --store ~/.research_b200/sessions --port 8765

With ``--project DIR`` the evaluation dev loop of that folder is served under ``/api/dev`` (configs, dataset previews,
config generation, launching / following / stopping runs, results): see ``frontend/devloop.py``.

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


DEV_PAGE = """<!doctype html><meta charset="utf-8"><title>evaluation dev loop</title>
<style>body{font-family:system-ui;margin:1.5rem;display:grid;grid-template-columns:18rem 1fr;gap:1.5rem}h2{font-size:1rem;margin:.8rem 0 .3rem}
li{cursor:pointer;list-style:none;padding:.15rem .3rem}li:hover{background:#eef}ul{padding:0;margin:0}pre{background:#f6f6f6;padding:.6rem;
overflow:auto;max-height:70vh;white-space:pre-wrap}button{margin-right:.4rem}.st{color:#777;font-size:.85em}</style>
<nav><h2>configs</h2><ul id="configs"></ul><h2>runs</h2><ul id="runs"></ul><h2>results</h2><ul id="traces"></ul><h2>datasets</h2><ul id="datasets"></ul></nav>
<main><div id="actions"></div><pre id="view">pick a config, a run, a result or a dataset</pre></main>
<script>
const $=id=>document.getElementById(id), view=$('view'), J=async(u,o)=>(await fetch(u,o)).json();
let es=null; const show=(t,a='')=>{if(es){es.close();es=null}$('actions').innerHTML=a;view.textContent=t};
const item=(ul,text,fn)=>{const li=document.createElement('li');li.textContent=text;li.onclick=fn;$(ul).appendChild(li)};
async function refresh(){for(const id of ['configs','runs','traces','datasets'])$(id).innerHTML='';
 for(const c of await J('/api/dev/configs'))item('configs',c.name,()=>openConfig(c.name));
 for(const r of await J('/api/dev/runs'))item('runs',r.config_name+' · '+r.status,()=>follow(r.run_id));
 for(const t of await J('/api/dev/traces'))item('traces',t.id+(t.summary.mean_reward!==undefined?' · '+t.summary.mean_reward.toFixed(3):''),()=>openTrace(t.id));
 for(const d of await J('/api/dev/datasets'))item('datasets',d.path,async()=>show(JSON.stringify(await J('/api/dev/dataset?path='+encodeURIComponent(d.path)),null,1)))}
async function openConfig(n){const c=await J('/api/dev/config/'+n);show(c.source,'<button id=go>launch</button><span class=st>'+(c.doc||'').split('\\n')[0]+'</span>');
 $('go').onclick=async()=>{const r=await J('/api/dev/launch/'+n,{method:'POST'});await refresh();follow(r.run_id)}}
function follow(id){show('','<button id=kill>stop</button><span class=st>'+id+'</span>');$('kill').onclick=()=>fetch('/api/dev/run/'+id+'/kill',{method:'POST'});
 es=new EventSource('/api/dev/run/'+id+'/stream');es.onmessage=e=>{view.textContent+=JSON.parse(e.data)+'\\n';view.scrollTop=view.scrollHeight};
 es.addEventListener('done',e=>{view.textContent+='\\n['+e.data+']';es.close();es=null;refresh()})}
async function openTrace(id){const t=await J('/api/dev/trace/'+id);show(JSON.stringify(t.summary,null,1)+'\\n\\n'+t.samples.map(s=>JSON.stringify(s)).join('\\n'))}
refresh();
</script>"""


def _mount_devloop(app, dev) -> None:
    """``/api/dev/*``: the evaluation dev loop of one project folder (``frontend/devloop.py``)."""
    import asyncio
    import json

    from fastapi import HTTPException
    from fastapi.responses import StreamingResponse

    def guarded(fn, *a, **kw):
        try:
            return fn(*a, **kw)
        except (FileNotFoundError, KeyError) as e:
            raise HTTPException(404, str(e)) from e
        except FileExistsError as e:
            raise HTTPException(409, str(e)) from e
        except (ValueError, SyntaxError) as e:
            raise HTTPException(400, str(e)) from e

    from fastapi.responses import HTMLResponse

    @app.get("/dev", response_class=HTMLResponse)
    async def dev_page():
        return DEV_PAGE

    @app.get("/api/dev/configs")
    async def configs():
        return dev.list_configs()

    @app.get("/api/dev/config/{name}")
    async def config(name: str):
        return guarded(dev.load_config, name)

    @app.get("/api/dev/config/{name}/dataset")
    async def config_dataset(name: str, n: int = 5):
        return guarded(dev.dataset_preview_for_config, name, n)

    @app.post("/api/dev/generate")
    async def generate(body: dict):
        """Form fields (or ``source``) -> config source; with ``save`` it is written to ``configs/`` under a numbered name."""
        from .devloop import generate_config

        if body.get("save"):
            return guarded(dev.save_config, body, body.get("name"), bool(body.get("overwrite")))
        return {"source": guarded(generate_config, body)}

    @app.get("/api/dev/datasets")
    async def datasets():
        return dev.list_datasets()

    @app.get("/api/dev/dataset")
    async def dataset(path: str, n: int = 5):
        return guarded(dev.preview, path, n)

    @app.get("/api/dev/models")
    async def models():
        return dev.list_models()

    @app.get("/api/dev/traces")
    async def traces():
        return dev.list_traces()

    @app.get("/api/dev/trace/{trace_id}")
    async def trace(trace_id: str, limit: int = 200):
        return guarded(dev.get_trace, trace_id, limit)

    @app.post("/api/dev/launch/{name}")
    async def launch(name: str, body: dict | None = None):
        return guarded(dev.launch, name, list((body or {}).get("args", [])))

    @app.get("/api/dev/runs")
    async def runs():
        return dev.runs.list()

    @app.get("/api/dev/run/{run_id}/output")
    async def run_output(run_id: str, since: int = 0):
        return guarded(dev.runs.output, run_id, since)

    @app.get("/api/dev/run/{run_id}/stream")
    async def run_stream(run_id: str, since: int = 0):
        """Server-sent events: one ``data:`` line per output line, then ``event: done`` with the exit code."""
        guarded(dev.runs.output, run_id, since)

        async def events():
            at = since
            while True:
                chunk = dev.runs.output(run_id, at)
                for line in chunk["lines"]:
                    yield f"data: {json.dumps(line)}\n\n"
                at = chunk["next"]
                if chunk["done"]:
                    yield f"event: done\ndata: {json.dumps({'status': chunk['status'], 'exit_code': chunk['exit_code']})}\n\n"
                    return
                await asyncio.sleep(0.2)

        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/api/dev/run/{run_id}/kill")
    async def run_kill(run_id: str):
        return {"killed": await asyncio.to_thread(guarded, dev.runs.kill, run_id)}

    @app.delete("/api/dev/run/{run_id}")
    async def run_delete(run_id: str):
        if not dev.runs.delete(run_id):
            raise HTTPException(409, "no such run, or it is still running")
        return {"deleted": run_id}


def create_app(store: FileSessionStore, rollout_override=None, devloop=None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import HTMLResponse

    app = FastAPI(title="research_b200 sessions")
    if devloop is not None:
        _mount_devloop(app, devloop)

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
    ap.add_argument("--project", default="", help="project folder (configs/, data/, results/) for the evaluation dev loop under /api/dev")
    args = ap.parse_args()
    dev = None
    if args.project:
        from .devloop import DevLoop

        dev = DevLoop(args.project)
    uvicorn.run(create_app(FileSessionStore(args.store), devloop=dev), host=args.host, port=args.port, log_level="warning")


if __name__ == "__main__":
    main()
