"""Live training report over HTTP (the reference's ``librembrandt_reportserv`` side crate: an HTTP server on
127.0.0.1:8080 with a plotting page at ``/`` and a JSON series at ``/api/v0/train_loss.json``; there the JSON is a
canned series and the server is not wired to the trainer, librembrandt_reportserv/src/lib.rs:52-161).

Here the server is fed by ``SgdOpt`` (``report=ReportServer(...)``) and serves the real series. The page draws in
the browser with a few lines of canvas code; nothing is rendered on the training machine.
"""
from __future__ import annotations

import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>rembrandt-b200 report</title>
<style>body{font-family:sans-serif;margin:2em}canvas{border:1px solid #ccc}</style></head><body>
<h2>training loss</h2><canvas id="c" width="900" height="360"></canvas>
<p id="s"></p>
<script>
async function draw(){
  const r = await fetch('/api/v0/train_loss.json'); const d = await r.json();
  const c = document.getElementById('c'), g = c.getContext('2d'); g.clearRect(0,0,c.width,c.height);
  const pts = d.train_loss; if(!pts.length){return;}
  const xs = pts.map(p=>p[0]), ys = pts.map(p=>p[1]);
  const x0=Math.min(...xs), x1=Math.max(...xs,x0+1), y0=0, y1=Math.max(...ys,1e-9);
  g.beginPath();
  pts.forEach((p,i)=>{const x=(p[0]-x0)/(x1-x0)*(c.width-20)+10, y=c.height-10-(p[1]-y0)/(y1-y0)*(c.height-20);
    if(i==0) g.moveTo(x,y); else g.lineTo(x,y);});
  g.strokeStyle='#06c'; g.stroke();
  const v = d.valid_accuracy; document.getElementById('s').textContent =
    'iterations: '+x1+'  last loss: '+ys[ys.length-1].toFixed(4)+(v.length?('  last validation accuracy: '+v[v.length-1][1].toFixed(4)):'');
}
draw(); setInterval(draw, 2000);
</script></body></html>"""


class ReportServerState:
    def __init__(self):
        self.lock = threading.Lock()
        self.train_loss, self.train_accuracy, self.valid_loss, self.valid_accuracy = [], [], [], []

    def update_training(self, t, loss, accuracy):
        with self.lock:
            self.train_loss.append((int(t), float(loss)))
            self.train_accuracy.append((int(t), float(accuracy)))

    def update_validation(self, t, loss, accuracy):
        with self.lock:
            self.valid_loss.append((int(t), float(loss)))
            self.valid_accuracy.append((int(t), float(accuracy)))

    def as_json(self):
        with self.lock:
            return json.dumps({"train_loss": self.train_loss, "train_accuracy": self.train_accuracy,
                               "valid_loss": self.valid_loss, "valid_accuracy": self.valid_accuracy})


class ReportServer(ReportServerState):
    def __init__(self, host="127.0.0.1", port=8080):
        super().__init__()
        state = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):
                if self.path == "/":
                    body, ctype = _PAGE.encode(), "text/html; charset=utf-8"
                elif self.path.startswith("/api/v0/train_loss.json"):
                    body, ctype = state.as_json().encode(), "application/json"
                else:
                    self.send_error(404)
                    return
                self.send_response(200)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.thread.start()

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()
