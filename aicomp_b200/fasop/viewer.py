"""Small web viewer for FASOP results: ``python -m aicomp_b200.fasop.viewer --log main_logs/x.jsonl --port 8050``.

Serves one page (stdlib ``http.server``, no external assets) that polls the JSON-lines file a search writes and
draws the time/cost scatter with the Pareto front plus a sortable table; ``POST /run`` starts a new search with the
posted arguments.  Role of the reference's ``fasop/demo/web_pareto_viewer.py`` (Plotly page that tails the JSONL
stream and can spawn ``FASOP.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>FASOP B200</title>
<style>body{font-family:sans-serif;margin:1.5em}table{border-collapse:collapse;font-size:12px}td,th{border:1px solid #ccc;padding:2px 6px}
th{cursor:pointer;background:#eee}.oom{color:#b00}svg{border:1px solid #ccc}</style></head><body>
<h2>FASOP strategy search</h2><div id="meta"></div>
<svg id="plot" width="720" height="360"></svg>
<table id="tbl"><thead></thead><tbody></tbody></table>
<script>
let rows=[],sortKey='total_time',asc=true;
const cols=['rank','gbs','mbs','tp','dp','pp','step_time','throughput','oom_gpumem','is_oom','cost','partition'];
function pareto(r){const p=r.filter(x=>!x.is_oom).sort((a,b)=>a.total_time-b.total_time);let best=1e99,f=[];for(const x of p){if(x.cost<best){f.push(x);best=x.cost}}return f}
function draw(){const s=document.getElementById('plot');s.innerHTML='';const ok=rows.filter(x=>!x.is_oom);if(!ok.length)return;
const xs=ok.map(r=>r.total_time),ys=ok.map(r=>r.cost),x0=Math.min(...xs),x1=Math.max(...xs),y0=Math.min(...ys),y1=Math.max(...ys);
const X=v=>40+(v-x0)/(x1-x0+1e-9)*660,Y=v=>340-(v-y0)/(y1-y0+1e-9)*320;
for(const r of ok){const c=document.createElementNS('http://www.w3.org/2000/svg','circle');c.setAttribute('cx',X(r.total_time));c.setAttribute('cy',Y(r.cost));c.setAttribute('r',3);c.setAttribute('fill','#48a');
const t=document.createElementNS('http://www.w3.org/2000/svg','title');t.textContent=`tp${r.tp} dp${r.dp} pp${r.pp} mbs${r.mbs}: ${r.step_time.toFixed(3)} s/step`;c.appendChild(t);s.appendChild(c)}
const f=pareto(rows);if(f.length){const pl=document.createElementNS('http://www.w3.org/2000/svg','polyline');pl.setAttribute('points',f.map(r=>X(r.total_time)+','+Y(r.cost)).join(' '));pl.setAttribute('fill','none');pl.setAttribute('stroke','#d40');s.appendChild(pl)}}
function table(){const th=document.querySelector('#tbl thead'),tb=document.querySelector('#tbl tbody');
th.innerHTML='<tr>'+cols.map(c=>`<th onclick="sortBy('${c}')">${c}</th>`).join('')+'</tr>';
const r=[...rows].sort((a,b)=>(a[sortKey]>b[sortKey]?1:-1)*(asc?1:-1));
tb.innerHTML=r.map(x=>'<tr class="'+(x.is_oom?'oom':'')+'">'+cols.map(c=>'<td>'+(typeof x[c]=='number'&&!Number.isInteger(x[c])?x[c].toFixed(4):JSON.stringify(x[c]))+'</td>').join('')+'</tr>').join('')}
function sortBy(k){asc=(sortKey==k)?!asc:true;sortKey=k;table()}
async function poll(){const j=await (await fetch('/data')).json();rows=j.rows;document.getElementById('meta').textContent=JSON.stringify(j.meta);draw();table();setTimeout(poll,2000)}
poll();
</script></body></html>"""


def read_log(path: str):
    meta, rows = {}, []
    if path and os.path.exists(path):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                try:
                    o = json.loads(line)
                except json.JSONDecodeError:
                    continue  # a line still being written
                if o.get("type") == "meta":
                    meta = o
                else:
                    rows.append(o)
    ok = sorted([r for r in rows if not r.get("is_oom")], key=lambda r: r["total_time"])
    for i, r in enumerate(ok + [r for r in rows if r.get("is_oom")]):
        r["rank"] = i + 1
    return meta, rows


def make_handler(state):
    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _send(self, code, body, ctype):
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path.startswith("/data"):
                meta, rows = read_log(state["log"])
                self._send(200, json.dumps({"meta": meta, "rows": rows}).encode(), "application/json")
            else:
                self._send(200, PAGE.encode(), "text/html; charset=utf-8")

        def do_POST(self):
            if self.path != "/run":
                return self._send(404, b"", "text/plain")
            n = int(self.headers.get("Content-Length", "0"))
            args = json.loads(self.rfile.read(n) or b"{}").get("args", [])
            if not all(isinstance(x, str) for x in args):
                return self._send(400, b"args must be strings", "text/plain")
            state["proc"] = subprocess.Popen([sys.executable, "-m", "aicomp_b200.fasop", *args], cwd=state["cwd"])
            self._send(202, b"started", "text/plain")
    return H


def serve(log: str, port: int = 8050, host: str = "127.0.0.1"):
    state = {"log": log, "proc": None, "cwd": os.getcwd()}
    srv = ThreadingHTTPServer((host, port), make_handler(state))
    return srv, state


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--log", required=True)
    ap.add_argument("--port", type=int, default=8050)
    ap.add_argument("--host", default="127.0.0.1")
    a = ap.parse_args(argv)
    srv, _ = serve(a.log, a.port, a.host)
    print(f"FASOP viewer on http://{a.host}:{a.port}/  (log: {a.log})")
    srv.serve_forever()


if __name__ == "__main__":
    main()
