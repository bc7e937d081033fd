"""The built-in chat page served at ``/`` (single static document, no build step): streaming chat against
``/v1/chat/completions`` with a collapsible thinking block, conversations kept in the browser's
localStorage, sampling settings, and image attachment as data URLs (``web/`` in the reference)."""

INDEX_HTML = r"""<!doctype html>
<html lang="en"><head><meta charset="utf-8"><meta name="viewport" content="width=device-width,initial-scale=1">
<title>legion-b200</title>
<style>
:root{color-scheme:light dark;--bg:#111;--fg:#eee;--mut:#888;--acc:#4da3ff;--card:#1c1c1c}
@media(prefers-color-scheme:light){:root{--bg:#fafafa;--fg:#111;--mut:#666;--card:#fff}}
*{box-sizing:border-box}body{margin:0;font:15px/1.5 system-ui,sans-serif;background:var(--bg);color:var(--fg);display:flex;height:100vh}
#side{width:230px;border-right:1px solid #3334;padding:10px;overflow:auto}#side button{width:100%;margin-bottom:8px}
.conv{padding:6px 8px;border-radius:6px;cursor:pointer;white-space:nowrap;overflow:hidden;text-overflow:ellipsis}.conv.on{background:var(--card)}
#main{flex:1;display:flex;flex-direction:column;min-width:0}#log{flex:1;overflow:auto;padding:16px}
.msg{max-width:820px;margin:0 auto 14px;padding:10px 14px;border-radius:10px;background:var(--card);white-space:pre-wrap;word-wrap:break-word}
.msg.user{border-left:3px solid var(--acc)}.think{color:var(--mut);font-size:13px;border-left:2px solid #5556;padding-left:8px;margin-bottom:6px}
.meta{color:var(--mut);font-size:12px;margin-top:6px}#bar{display:flex;gap:8px;padding:12px;border-top:1px solid #3334;max-width:860px;width:100%;margin:0 auto}
textarea{flex:1;resize:none;height:64px;padding:8px;border-radius:8px;border:1px solid #5556;background:var(--card);color:var(--fg);font:inherit}
button{padding:8px 14px;border-radius:8px;border:0;background:var(--acc);color:#fff;cursor:pointer}button.sec{background:#5555}
#settings{display:none;padding:10px 16px;border-top:1px solid #3334;font-size:13px}#settings label{margin-right:14px}
#settings input{width:70px}
</style></head><body>
<div id="side"><button id="new">New chat</button><div id="convs"></div></div>
<div id="main"><div id="log"></div>
<div id="settings"><label>temperature <input id="temp" type="number" step="0.1" min="0" max="2" value="0.7"></label>
<label>top_p <input id="topp" type="number" step="0.05" min="0" max="1" value="0.95"></label>
<label>max_tokens <input id="maxt" type="number" min="1" value="1024"></label>
<label><input id="think" type="checkbox" checked style="width:auto"> thinking</label>
<label>API key <input id="key" type="password" style="width:160px"></label></div>
<div id="bar"><textarea id="in" placeholder="Message (Enter to send, Shift+Enter for a new line)"></textarea>
<input id="file" type="file" accept="image/*" style="display:none"><button class="sec" id="img" title="attach image">+</button>
<button class="sec" id="cfg">&#9881;</button><button id="send">Send</button></div></div>
<script>
const $=id=>document.getElementById(id);let convs=JSON.parse(localStorage.getItem('legion.convs')||'[]'),cur=null,busy=null,pendingImg=null;
function save(){localStorage.setItem('legion.convs',JSON.stringify(convs))}
function esc(s){return s.replace(/[&<>]/g,c=>({'&':'&amp;','<':'&lt;','>':'&gt;'}[c]))}
function renderSide(){$('convs').innerHTML='';convs.forEach((c,i)=>{const d=document.createElement('div');d.className='conv'+(c===cur?' on':'');d.textContent=c.title||'New chat';d.onclick=()=>{cur=c;render()};d.ondblclick=()=>{convs.splice(i,1);if(cur===c)cur=null;save();render()};$('convs').appendChild(d)})}
function render(){renderSide();$('log').innerHTML='';if(!cur)return;cur.msgs.forEach(m=>{const d=document.createElement('div');d.className='msg '+m.role;let h='';if(m.thinking)h+='<details class="think"><summary>thinking</summary>'+esc(m.thinking)+'</details>';h+=esc(typeof m.content==='string'?m.content:m.content.filter(p=>p.type==='text').map(p=>p.text).join(''));if(m.meta)h+='<div class="meta">'+esc(m.meta)+'</div>';d.innerHTML=h;$('log').appendChild(d)});$('log').scrollTop=1e9}
async function send(){if(busy){busy.abort();return}const text=$('in').value.trim();if(!text)return;if(!cur){cur={title:text.slice(0,40),msgs:[]};convs.unshift(cur)}
let content=text;if(pendingImg){content=[{type:'text',text},{type:'image_url',image_url:{url:pendingImg}}];pendingImg=null}
cur.msgs.push({role:'user',content});const a={role:'assistant',content:'',thinking:''};cur.msgs.push(a);$('in').value='';render();
busy=new AbortController();$('send').textContent='Stop';const t0=performance.now();let n=0;
try{const h={'content-type':'application/json'};if($('key').value)h.authorization='Bearer '+$('key').value;
const r=await fetch('/v1/chat/completions',{method:'POST',headers:h,signal:busy.signal,body:JSON.stringify({model:'default',stream:true,stream_options:{include_usage:true},
messages:cur.msgs.slice(0,-1).map(m=>({role:m.role,content:m.content})),temperature:+$('temp').value,top_p:+$('topp').value,max_tokens:+$('maxt').value,chat_template_kwargs:{enable_thinking:$('think').checked}})});
if(!r.ok){a.content='[error '+r.status+'] '+await r.text();}else{const rd=r.body.getReader(),dec=new TextDecoder();let buf='';
for(;;){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value,{stream:true});let i;while((i=buf.indexOf('\n\n'))>=0){const line=buf.slice(0,i);buf=buf.slice(i+2);if(!line.startsWith('data: '))continue;const p=line.slice(6);if(p==='[DONE]')continue;
const j=JSON.parse(p);const d=j.choices&&j.choices[0]&&j.choices[0].delta;if(d){if(d.content){a.content+=d.content;n++}if(d.reasoning_content){a.thinking+=d.reasoning_content;n++}}
if(j.usage)a.meta=j.usage.completion_tokens+' tokens, '+(j.usage.completion_tokens/((performance.now()-t0)/1000)).toFixed(1)+' tok/s';render()}}}}
catch(e){if(e.name!=='AbortError')a.content+='\n[error] '+e}
busy=null;$('send').textContent='Send';save();render()}
$('send').onclick=send;$('in').onkeydown=e=>{if(e.key==='Enter'&&!e.shiftKey){e.preventDefault();send()}};
$('new').onclick=()=>{cur=null;render()};$('cfg').onclick=()=>{const s=$('settings');s.style.display=s.style.display==='block'?'none':'block'};
$('img').onclick=()=>$('file').click();$('file').onchange=e=>{const f=e.target.files[0];if(!f)return;const r=new FileReader();r.onload=()=>{pendingImg=r.result};r.readAsDataURL(f)};
render();
</script></body></html>
"""
