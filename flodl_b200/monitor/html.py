"""Self-contained HTML pages (inline JS, no external assets) for the training dashboard and the
timeline viewer."""
from __future__ import annotations

import json

_STYLE = """
body{font-family:system-ui,sans-serif;margin:0;background:#14161a;color:#dde}
header{padding:12px 20px;background:#1d2026;border-bottom:1px solid #333}
h1{font-size:16px;margin:0} .sub{color:#8a93a6;font-size:12px}
main{padding:16px 20px;display:grid;grid-template-columns:repeat(auto-fit,minmax(420px,1fr));gap:16px}
.card{background:#1d2026;border:1px solid #2c3038;border-radius:6px;padding:12px}
canvas{width:100%;height:220px} table{border-collapse:collapse;width:100%;font-size:12px}
td,th{padding:3px 8px;border-bottom:1px solid #2c3038;text-align:right} th{color:#8a93a6}
#svg svg{max-width:100%;height:auto;background:#fff;border-radius:4px}
"""

_PLOT_JS = """
function plot(canvas, series, names){
  const c=canvas.getContext('2d');const W=canvas.width=canvas.clientWidth*2,H=canvas.height=canvas.clientHeight*2;
  c.clearRect(0,0,W,H);c.lineWidth=2;c.font='20px system-ui';
  const colors=['#6cf','#fc6','#9e6','#f7a','#c9f','#6fc','#fa6','#aaa'];
  let lo=Infinity,hi=-Infinity,n=0;series.forEach(s=>{s.forEach(v=>{if(v!=null&&isFinite(v)){lo=Math.min(lo,v);hi=Math.max(hi,v)}});n=Math.max(n,s.length)});
  if(!isFinite(lo)){return} if(hi==lo){hi=lo+1}
  c.strokeStyle='#333';c.strokeRect(60,10,W-70,H-50);c.fillStyle='#8a93a6';
  c.fillText(hi.toPrecision(4),2,24);c.fillText(lo.toPrecision(4),2,H-44);
  series.forEach((s,k)=>{c.strokeStyle=colors[k%8];c.beginPath();let started=false;
    s.forEach((v,i)=>{if(v==null)return;const x=60+(W-70)*(n>1?i/(n-1):0.5),y=10+(H-60)*(1-(v-lo)/(hi-lo));
      if(started)c.lineTo(x,y);else{c.moveTo(x,y);started=true}});c.stroke();
    c.fillStyle=colors[k%8];c.fillText(names[k]||'',70+k*160,H-12)});
}
"""


def dashboard_html(state: dict, live: bool) -> str:
    """`state`: {total_epochs, epochs:[{epoch,duration_secs,metrics,resources}], svg, label, hash, hardware, metadata}."""
    return f"""<!doctype html><html><head><meta charset="utf-8"><title>training monitor</title><style>{_STYLE}</style></head>
<body><header><h1 id="title">training</h1><div class="sub" id="sub"></div></header>
<main><div class="card"><canvas id="metrics"></canvas></div><div class="card"><canvas id="res"></canvas></div>
<div class="card"><table id="tbl"></table></div><div class="card" id="svg"></div><div class="card"><pre id="meta" style="font-size:11px"></pre></div></main>
<script>{_PLOT_JS}
let S={json.dumps(state)};const LIVE={'true' if live else 'false'};
function render(){{
  document.getElementById('title').textContent=(S.label||'training')+(S.hash?' ['+S.hash.slice(0,8)+']':'');
  document.getElementById('sub').textContent=(S.hardware||'')+'  epochs '+S.epochs.length+'/'+S.total_epochs;
  const names=[];S.epochs.forEach(e=>Object.keys(e.metrics).forEach(k=>{{if(!names.includes(k))names.push(k)}}));
  plot(document.getElementById('metrics'),names.map(k=>S.epochs.map(e=>e.metrics[k]??null)),names);
  plot(document.getElementById('res'),[S.epochs.map(e=>e.resources.cpu_percent),S.epochs.map(e=>e.resources.gpu_util_percent)],['cpu %','gpu %']);
  let h='<tr><th>epoch</th><th>secs</th>'+names.map(n=>'<th>'+n+'</th>').join('')+'</tr>';
  S.epochs.slice(-30).forEach(e=>{{h+='<tr><td>'+(e.epoch+1)+'</td><td>'+e.duration_secs.toFixed(2)+'</td>'+names.map(n=>'<td>'+(e.metrics[n]??'').toString().slice(0,9)+'</td>').join('')+'</tr>'}});
  document.getElementById('tbl').innerHTML=h;
  if(S.svg)document.getElementById('svg').innerHTML=S.svg;
  document.getElementById('meta').textContent=S.metadata?JSON.stringify(S.metadata,null,1):'';
}}
render();
if(LIVE){{const es=new EventSource('/events');
  es.addEventListener('epoch',m=>{{S.epochs.push(JSON.parse(m.data));render()}});
  es.addEventListener('init',m=>{{const d=JSON.parse(m.data);Object.assign(S,d);render()}});}}
</script></body></html>"""


def timeline_html(data: dict) -> str:
    return f"""<!doctype html><html><head><meta charset="utf-8"><title>timeline</title><style>{_STYLE}</style></head>
<body><header><h1>timeline</h1><div class="sub" id="sub"></div></header>
<main><div class="card"><canvas id="gpu"></canvas></div><div class="card"><canvas id="cpu"></canvas></div>
<div class="card"><table id="ev"></table></div></main>
<script>{_PLOT_JS}
const D={json.dumps(data)};
const idx=[];D.samples.forEach(s=>s.gpus.forEach(g=>{{if(!idx.includes(g.index))idx.push(g.index)}}));
plot(document.getElementById('gpu'),idx.map(i=>D.samples.map(s=>{{const g=s.gpus.find(g=>g.index==i);return g?g.util:null}})),idx.map(i=>'GPU'+i+' %'));
plot(document.getElementById('cpu'),[D.samples.map(s=>s.cpu_percent)],['cpu %']);
document.getElementById('sub').textContent=D.samples.length+' samples, '+D.events.length+' events';
let h='<tr><th>t (ms)</th><th>event</th><th>detail</th></tr>';
D.events.slice(-200).forEach(e=>{{const d=Object.assign({{}},e);delete d.t_ms;delete d.kind;h+='<tr><td>'+e.t_ms+'</td><td>'+e.kind+'</td><td>'+JSON.stringify(d)+'</td></tr>'}});
document.getElementById('ev').innerHTML=h;
</script></body></html>"""
