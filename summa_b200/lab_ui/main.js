// Model lab front end: loads a trace (live from /api/trace, from a file, or the built-in demo)
// and draws tokens, next-token candidates, the block stack, attention heatmaps (canvas),
// residual-stream activity (canvas), the norm profile and training metrics (SVG).
(function () {
  'use strict';
  const U = window.TraceUtils;
  const $ = (id) => document.getElementById(id);
  const state = { trace: null, layer: 0, timer: null, hidden: new Set() };
  const SVG = 'http://www.w3.org/2000/svg';

  function showError(msg) {
    const e = $('error');
    e.hidden = !msg;
    e.textContent = msg || '';
  }

  // ---------------------------------------------------------------- loading
  async function refreshStatus() {
    try {
      const r = await fetch('/api/status');
      if (!r.ok) throw new Error(r.status);
      const s = await r.json();
      $('status').textContent = s.model + ' · ' + (s.parameters / 1e6).toFixed(1) + ' M parameters';
      $('status').className = 'pill ok';
    } catch (e) {
      $('status').textContent = 'offline (file / demo traces only)';
      $('status').className = 'pill off';
    }
  }

  async function traceLive(prompt) {
    showError('');
    try {
      const r = await fetch('/api/trace?prompt=' + encodeURIComponent(prompt));
      const body = await r.text();
      if (!r.ok) throw new Error(JSON.parse(body).error || r.status);
      setTrace(U.parseTraceJson(body));
    } catch (e) {
      showError('trace failed: ' + e.message);
    }
  }

  function setTrace(t) {
    state.trace = t;
    state.layer = 0;
    $('layer').max = Math.max(0, t.layers.length - 1);
    $('layer').value = 0;
    renderAll();
  }

  // ---------------------------------------------------------------- drawing helpers
  function heatmap(canvas, matrix, lo, hi) {
    const ctx = canvas.getContext('2d');
    const w = canvas.width, h = canvas.height;
    const rows = Math.min(matrix.length, h), cols = Math.min(matrix[0].length, w);
    const m = (rows === matrix.length && cols === matrix[0].length) ? matrix : U.resample(matrix, rows, cols);
    const img = ctx.createImageData(w, h);
    for (let y = 0; y < h; y++) {
      const r = Math.min(rows - 1, Math.floor((y * rows) / h));
      for (let x = 0; x < w; x++) {
        const c = Math.min(cols - 1, Math.floor((x * cols) / w));
        const [R, G, B] = U.colour((m[r][c] - lo) / (hi - lo));
        const o = 4 * (y * w + x);
        img.data[o] = R; img.data[o + 1] = G; img.data[o + 2] = B; img.data[o + 3] = 255;
      }
    }
    ctx.putImageData(img, 0, 0);
  }

  function el(name, attrs, parent) {
    const e = document.createElementNS(SVG, name);
    for (const [k, v] of Object.entries(attrs || {})) e.setAttribute(k, v);
    if (parent) parent.appendChild(e);
    return e;
  }

  function linePath(points, x0, x1, y0, y1, W, H, pad) {
    const sx = (x) => pad + ((x - x0) / (x1 - x0 || 1)) * (W - 2 * pad);
    const sy = (y) => H - pad - ((y - y0) / (y1 - y0 || 1)) * (H - 2 * pad);
    return points.map((p, i) => (i ? 'L' : 'M') + sx(p[0]).toFixed(1) + ' ' + sy(p[1]).toFixed(1)).join(' ');
  }

  const PALETTE = ['#e4572e', '#17bebb', '#ffc914', '#76b041', '#a37cf0', '#f28fbb', '#5b8def', '#9c9c9c'];

  // ---------------------------------------------------------------- panels
  function renderTokens(t) {
    const box = $('tokens');
    box.replaceChildren();
    t.tokens.forEach((tok, i) => {
      const s = document.createElement('span');
      s.className = 'tok';
      s.title = '#' + tok.original_index + ' id ' + tok.id + ' (' + tok.source + ')';
      s.textContent = tok.display === null || tok.display === undefined ? String(tok.id) : tok.display;
      if (tok.source === 'generated') s.className = 'tok generated';
      box.appendChild(s);
    });
    // the continuation the model produced and the sampling settings that produced it; per-token RMS of the
    // last stage as bars (the signal that reaches the output head)
    const c = $('candidates');
    c.replaceChildren();
    const head = document.createElement('div');
    const smp = t.sampling || {};
    head.textContent = 'generated: ' + JSON.stringify(t.generated_text || '') + '  (T ' + (smp.temperature ?? 0) +
      ', seed ' + (smp.seed ?? 0) + (t.capture && t.capture.tokens_truncated ? ', leading tokens dropped: ' +
      t.capture.dropped_leading_tokens : '') + ')';
    c.appendChild(head);
    const last = t.bundle.inference.stages[t.bundle.inference.stages.length - 1].token_rms;
    const top = Math.max(...last, 1e-9);
    last.slice(-10).forEach((v, i) => {
      const row = document.createElement('div');
      row.className = 'bar';
      const label = document.createElement('span');
      const tok = t.tokens[t.tokens.length - Math.min(10, last.length) + i];
      label.textContent = (tok ? tok.display : '') + '  rms ' + v.toFixed(3);
      const fill = document.createElement('i');
      fill.style.width = (100 * v / top).toFixed(1) + '%';
      row.append(fill, label);
      c.appendChild(row);
    });
  }

  function renderArchitecture(t) {
    const box = $('architecture');
    box.replaceChildren();
    const mk = (cls, text) => {
      const d = document.createElement('div');
      d.className = 'blk ' + cls;
      d.textContent = text;
      return d;
    };
    box.appendChild(mk('io', 'embedding ' + t.model.vocab_size + ' × ' + t.model.hidden_size));
    t.layers.forEach((l, i) => {
      const d = mk(l.mixer + (i === state.layer ? ' current' : ''), i + ' · ' + l.mixer);
      d.onclick = () => { state.layer = i; $('layer').value = i; renderLayer(); renderArchitecture(t); };
      box.appendChild(d);
    });
    box.appendChild(mk('io', 'norm + head'));
  }

  function renderLayer() {
    const t = state.trace;
    const l = t.layers[state.layer];
    $('layer-label').textContent = 'layer ' + state.layer + ' (' + l.mixer + ')';
    $('attention-title').textContent = l.attention ? 'Attention (layer ' + state.layer + ', ' + l.attention.length +
      ' of ' + l.total_heads + ' heads)' : 'Layer ' + state.layer + ' is a Mamba block: final recurrent state (rows: state, columns: channel bins)';
    const heads = $('heads');
    heads.replaceChildren();
    if (l.mamba_state) {
      const fig = document.createElement('figure');
      const c = document.createElement('canvas');
      c.width = 440; c.height = 220;
      const [slo, shi] = U.extent(l.mamba_state);
      heatmap(c, l.mamba_state, slo, shi);
      const cap = document.createElement('figcaption');
      cap.textContent = 'recurrent state after the last token';
      fig.append(c, cap);
      heads.appendChild(fig);
    }
    (l.attention || []).forEach((h, j) => {
      const fig = document.createElement('figure');
      const c = document.createElement('canvas');
      c.width = c.height = 220;
      heatmap(c, h, 0, 1);
      const cap = document.createElement('figcaption');
      cap.textContent = 'head ' + j + ' (rows: queries, columns: keys)';
      fig.append(c, cap);
      heads.appendChild(fig);
    });
    // channels: tokens on x, channel bins on y
    const n = l.channels.length, bins = l.channels[0].length;
    const m = [];
    for (let b = 0; b < bins; b++) m.push(l.channels.map((row) => row[b]));
    const [lo, hi] = U.extent(m);
    heatmap($('channels'), m, lo, hi);
  }

  function renderNorms(t) {
    const svg = $('norms');
    svg.replaceChildren();
    const prof = U.layerNormProfile(t).map((v, i) => [i, v]);
    const ys = prof.map((p) => p[1]);
    const y1 = Math.max(...ys) * 1.05 || 1;
    el('path', { d: linePath(prof, 0, Math.max(1, prof.length - 1), 0, y1, 900, 180, 24), class: 'line', stroke: PALETTE[1] }, svg);
    prof.forEach((p) => {
      const x = 24 + (p[0] / Math.max(1, prof.length - 1)) * (900 - 48), y = 180 - 24 - (p[1] / y1) * (180 - 48);
      el('circle', { cx: x, cy: y, r: p[0] === state.layer ? 6 : 3, fill: PALETTE[p[0] === state.layer ? 0 : 1] }, svg);
    });
    el('text', { x: 28, y: 16, class: 'axis' }, svg).textContent = 'mean residual norm per layer (max ' + y1.toFixed(2) + ')';
  }

  function renderMetrics(t) {
    const svg = $('metrics'), legend = $('metric-legend');
    svg.replaceChildren();
    legend.replaceChildren();
    const series = U.metricSeries(t.metrics);
    const names = Object.keys(series).sort();
    if (!names.length) {
      el('text', { x: 28, y: 110, class: 'axis' }, svg).textContent = 'no metrics.jsonl records in this trace';
      return;
    }
    names.forEach((name, i) => {
      const colour = PALETTE[i % PALETTE.length];
      const b = document.createElement('button');
      b.type = 'button';
      b.textContent = name;
      b.style.borderColor = colour;
      b.className = state.hidden.has(name) ? 'off' : '';
      b.onclick = () => { state.hidden.has(name) ? state.hidden.delete(name) : state.hidden.add(name); renderMetrics(t); };
      legend.appendChild(b);
      if (state.hidden.has(name)) return;
      const pts = series[name];
      const xs = pts.map((p) => p[0]), ys = pts.map((p) => p[1]);
      // every series is normalised to its own range: the plot compares shapes, the legend names them
      el('path', { d: linePath(pts, Math.min(...xs), Math.max(...xs), Math.min(...ys), Math.max(...ys), 900, 220, 24),
        class: 'line', stroke: colour }, svg).appendChild(document.createElementNS(SVG, 'title')).textContent =
        name + ': ' + ys[0].toPrecision(4) + ' → ' + ys[ys.length - 1].toPrecision(4);
    });
  }

  function renderAll() {
    const t = state.trace;
    if (!t) return;
    renderTokens(t);
    renderArchitecture(t);
    renderLayer();
    renderNorms(t);
    renderMetrics(t);
  }

  // ---------------------------------------------------------------- events
  $('prompt-form').addEventListener('submit', (e) => {
    e.preventDefault();
    const p = $('prompt').value.trim();
    if (p) traceLive(p);
  });
  $('file').addEventListener('change', async (e) => {
    const f = e.target.files[0];
    if (!f) return;
    try { showError(''); setTrace(U.parseTraceJson(await f.text())); } catch (err) { showError(err.message); }
  });
  $('demo').addEventListener('click', () => { showError(''); setTrace(U.validateTrace(window.makeDemoTrace())); });
  $('layer').addEventListener('input', (e) => {
    state.layer = Number(e.target.value);
    renderLayer(); renderArchitecture(state.trace); renderNorms(state.trace);
  });
  $('play').addEventListener('click', () => {
    if (state.timer) { clearInterval(state.timer); state.timer = null; $('play').textContent = '▶ play stages'; return; }
    if (!state.trace) return;
    $('play').textContent = '■ stop';
    state.timer = setInterval(() => {
      state.layer = (state.layer + 1) % state.trace.layers.length;
      $('layer').value = state.layer;
      renderLayer(); renderArchitecture(state.trace); renderNorms(state.trace);
    }, 700);
  });

  refreshStatus();
  setTrace(U.validateTrace(window.makeDemoTrace()));
})();
