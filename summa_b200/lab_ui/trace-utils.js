// Trace validation and data shaping for the model lab. Works in a browser (attached to
// `window.TraceUtils`) and under node (`module.exports`), so the same file is unit-tested.
(function (root) {
  'use strict';

  const FORMAT = 'summa_model_trace';
  const MAX_TOKENS = 128;

  function fail(msg) { throw new Error('invalid trace: ' + msg); }
  function isNum(x) { return typeof x === 'number' && Number.isFinite(x); }

  function checkHeatmap(h, where) {
    if (!h || !Number.isInteger(h.rows) || !Number.isInteger(h.cols)) fail(where + ' heat-map header');
    if (!Array.isArray(h.values) || h.values.length !== h.rows * h.cols || !h.values.every(isNum)) fail(where + ' heat-map values');
    if (!Array.isArray(h.row_labels) || h.row_labels.length !== h.rows) fail(where + ' row labels');
    if (!Array.isArray(h.col_labels) || h.col_labels.length !== h.cols) fail(where + ' column labels');
  }

  // flat row-major heat-map -> array of rows
  function matrixOf(h) {
    const out = [];
    for (let r = 0; r < h.rows; r++) out.push(h.values.slice(r * h.cols, (r + 1) * h.cols));
    return out;
  }

  // Validates a `summa_model_trace` bundle (kind / version, model header with one architecture entry per
  // layer, token rows, stages = embedding + one block per layer + final_norm, rectangular heat-maps with
  // one row per captured token) and returns the view the renderers draw from:
  //   { model, tokens, layers: [{mixer, residual_norm, delta_norm, channels, attention?, mamba_state?}],
  //     embedding, final_norm, generated_text, metrics, capture, bundle }
  function validateTrace(t) {
    if (!t || typeof t !== 'object') fail('not an object');
    if (t.kind !== FORMAT) fail('kind must be ' + FORMAT);
    if (t.version !== 1) fail('unsupported version ' + t.version);
    const m = t.model;
    if (!m || typeof m.name !== 'string' || !Number.isInteger(m.num_layers)) fail('model header');
    if (!Array.isArray(m.layers) || m.layers.length !== m.num_layers) fail('model.layers must have one entry per layer');
    const inf = t.inference;
    if (!inf || !Array.isArray(inf.tokens) || inf.tokens.length === 0) fail('token count');
    const n = inf.tokens.length;
    if (!t.capture || t.capture.captured_tokens !== n) fail('capture.captured_tokens');
    inf.tokens.forEach((tok, i) => {
      if (!Number.isInteger(tok.id)) fail('token ' + i + ' has no id');
      if (tok.source !== 'prompt' && tok.source !== 'generated') fail('token ' + i + ' source');
    });
    const st = inf.stages;
    if (!Array.isArray(st) || st.length !== m.num_layers + 2) fail('stages');
    if (st[0].stage !== 'embedding' || st[st.length - 1].stage !== 'final_norm') fail('stage order');
    const layers = [];
    st.forEach((s, i) => {
      checkHeatmap(s.activation, 'stage ' + i);
      if (s.activation.rows !== n) fail('stage ' + i + ' rows');
      if (!Array.isArray(s.token_rms) || s.token_rms.length !== n || !s.token_rms.every(isNum)) fail('stage ' + i + ' token_rms');
      if (s.stage !== 'block') return;
      if (s.mixer !== 'attention' && s.mixer !== 'mamba') fail('stage ' + i + ' mixer');
      const layer = { mixer: s.mixer, label: s.label, residual_norm: s.token_rms, delta_norm: s.token_delta_rms || null,
                      channels: matrixOf(s.activation), stats: s.stats };
      if (s.attention) {
        if (!Array.isArray(s.attention.heads)) fail('stage ' + i + ' attention');
        s.attention.heads.forEach((h, j) => {
          checkHeatmap(h, 'stage ' + i + ' head ' + j);
          if (h.rows !== n || h.cols !== n) fail('stage ' + i + ' head ' + j + ' shape');
        });
        layer.attention = s.attention.heads.map(matrixOf);
        layer.total_heads = s.attention.total_heads;
      }
      if (s.mamba_state) {
        checkHeatmap(s.mamba_state, 'stage ' + i + ' mamba_state');
        layer.mamba_state = matrixOf(s.mamba_state);
      }
      layers.push(layer);
    });
    if (t.training !== undefined && (!t.training || !Array.isArray(t.training.rows))) fail('training.rows');
    return {
      model: m, tokens: inf.tokens, layers,
      embedding: matrixOf(st[0].activation), final_norm: matrixOf(st[st.length - 1].activation),
      prompt: inf.prompt, generated_text: inf.generated_text, sampling: inf.sampling,
      metrics: t.training ? t.training.rows : [], capture: t.capture, bundle: t,
    };
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
  // optimization / throughput / post_training_update events.
  function metricSeries(records) {
    const series = {};
    for (const rec of records || []) {
      const ev = rec && rec.event;
      if (!ev || !ev.values) continue;
      if (!['optimization', 'throughput', 'post_training_update'].includes(ev.type)) continue;
      for (const [k, v] of Object.entries(ev.values)) {
        if (!isNum(v)) continue;
        const name = ev.type === 'post_training_update' ? 'post.' + k : k;
        (series[name] = series[name] || []).push([rec.global_step || 0, v]);
      }
    }
    return series;
  }

  // per-layer mean of the residual norm: the "signal flow" line
  function layerNormProfile(trace) {
    return trace.layers.map((l) => l.residual_norm.reduce((a, b) => a + b, 0) / l.residual_norm.length);
  }

  const api = { FORMAT, MAX_TOKENS, matrixOf, validateTrace, parseTraceJson, resample, extent, colour, metricSeries, layerNormProfile };
  if (typeof module !== 'undefined' && module.exports) module.exports = api;
  else root.TraceUtils = api;
})(typeof window !== 'undefined' ? window : globalThis);
