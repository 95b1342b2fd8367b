// Trace validation and data shaping for the model lab. Works in a browser (attached to
// `window.TraceUtils`) and under node (`module.exports`), so the same file is unit-tested.
(function (root) {
  'use strict';

  const FORMAT = 'summa_model_trace';
  const MAX_TOKENS = 128;

  function fail(msg) { throw new Error('invalid trace: ' + msg); }
  function isNum(x) { return typeof x === 'number' && Number.isFinite(x); }

  // Throws on anything the renderers could not draw; returns the trace unchanged otherwise.
  function validateTrace(t) {
    if (!t || typeof t !== 'object') fail('not an object');
    if (t.format !== FORMAT) fail('format must be ' + FORMAT);
    if (t.version !== 1) fail('unsupported version ' + t.version);
    if (!t.model || typeof t.model.name !== 'string' || !Number.isInteger(t.model.num_layers)) fail('model header');
    if (!Array.isArray(t.tokens) || t.tokens.length === 0 || t.tokens.length > MAX_TOKENS) fail('token count');
    const n = t.tokens.length;
    t.tokens.forEach((tok, i) => { if (!Number.isInteger(tok.id)) fail('token ' + i + ' has no id'); });
    if (!Array.isArray(t.layers)) fail('layers');
    t.layers.forEach((l, i) => {
      if (l.mixer !== 'attention' && l.mixer !== 'ssm') fail('layer ' + i + ' mixer');
      if (!Array.isArray(l.residual_norm) || l.residual_norm.length !== n || !l.residual_norm.every(isNum)) {
        fail('layer ' + i + ' residual_norm');
      }
      if (!Array.isArray(l.channels) || l.channels.length !== n) fail('layer ' + i + ' channels');
      if (l.attention !== undefined) {
        if (!Array.isArray(l.attention)) fail('layer ' + i + ' attention');
        l.attention.forEach((h, j) => {
          if (!Array.isArray(h) || h.length !== n || !h.every((r) => Array.isArray(r) && r.length === n)) {
            fail('layer ' + i + ' head ' + j + ' shape');
          }
        });
      }
    });
    if (!Array.isArray(t.next_token)) fail('next_token');
    t.next_token.forEach((c) => { if (!Number.isInteger(c.id) || !isNum(c.probability)) fail('candidate'); });
    if (t.metrics !== undefined && !Array.isArray(t.metrics)) fail('metrics');
    return t;
  }

  function parseTraceJson(text) {
    let obj;
    try { obj = JSON.parse(text); } catch (e) { fail('not JSON (' + e.message + ')'); }
    return validateTrace(obj);
  }

  // Bilinear resampling of a row-major matrix onto (outRows x outCols); used when a heatmap has
  // more cells than pixels or fewer cells than a readable size.
  function resample(matrix, outRows, outCols) {
    const rows = matrix.length, cols = matrix[0].length;
    const out = [];
    for (let r = 0; r < outRows; r++) {
      const fr = rows === 1 ? 0 : (r * (rows - 1)) / Math.max(outRows - 1, 1);
      const r0 = Math.floor(fr), r1 = Math.min(r0 + 1, rows - 1), wr = fr - r0;
      const line = new Array(outCols);
      for (let c = 0; c < outCols; c++) {
        const fc = cols === 1 ? 0 : (c * (cols - 1)) / Math.max(outCols - 1, 1);
        const c0 = Math.floor(fc), c1 = Math.min(c0 + 1, cols - 1), wc = fc - c0;
        const top = matrix[r0][c0] * (1 - wc) + matrix[r0][c1] * wc;
        const bot = matrix[r1][c0] * (1 - wc) + matrix[r1][c1] * wc;
        line[c] = top * (1 - wr) + bot * wr;
      }
      out.push(line);
    }
    return out;
  }

  function extent(matrix) {
    let lo = Infinity, hi = -Infinity;
    for (const row of matrix) for (const v of row) { if (v < lo) lo = v; if (v > hi) hi = v; }
    if (!Number.isFinite(lo)) { lo = 0; hi = 1; }
    if (hi === lo) hi = lo + 1;
    return [lo, hi];
  }

  // value in [0, 1] -> [r, g, b]; dark blue -> teal -> yellow
  function colour(t) {
    const x = Math.min(1, Math.max(0, t));
    const stops = [[13, 8, 135], [36, 123, 160], [112, 193, 120], [253, 231, 37]];
    const f = x * (stops.length - 1), i = Math.min(Math.floor(f), stops.length - 2), w = f - i;
    return [0, 1, 2].map((k) => Math.round(stops[i][k] * (1 - w) + stops[i + 1][k] * w));
  }

  // metrics.jsonl records -> { name: [[global_step, value], ...] } for the numeric fields of
  // optimization / throughput / evaluation events.
  function metricSeries(records) {
    const series = {};
    for (const rec of records || []) {
      const ev = rec && rec.event;
      if (!ev || !ev.values) continue;
      if (!['optimization', 'throughput', 'evaluation'].includes(ev.type)) continue;
      for (const [k, v] of Object.entries(ev.values)) {
        if (!isNum(v)) continue;
        const name = ev.type === 'evaluation' ? 'eval.' + k : k;
        (series[name] = series[name] || []).push([rec.global_step || 0, v]);
      }
    }
    return series;
  }

  // per-layer mean of the residual norm: the "signal flow" line
  function layerNormProfile(trace) {
    return trace.layers.map((l) => l.residual_norm.reduce((a, b) => a + b, 0) / l.residual_norm.length);
  }

  const api = { FORMAT, MAX_TOKENS, validateTrace, parseTraceJson, resample, extent, colour, metricSeries, layerNormProfile };
  if (typeof module !== 'undefined' && module.exports) module.exports = api;
  else root.TraceUtils = api;
})(typeof window !== 'undefined' ? window : globalThis);
