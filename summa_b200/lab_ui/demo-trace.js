// A synthetic `summa_model_trace` bundle (no model needed): 12 tokens through a 6-block stack with one
// Mamba block, banded causal attention patterns and a decaying loss curve. Same shape as the bundles the
// `trace` command and `/api/trace` produce.
(function (root) {
  'use strict';
  function makeDemoTrace() {
    const words = ['The', ' quick', ' brown', ' fox', ' jumps', ' over', ' the', ' lazy', ' dog', ' and', ' runs', ' away'];
    const n = words.length, L = 6, bins = 32, prompt = 9;
    let seed = 7;
    const rnd = () => { seed = (seed * 1664525 + 1013904223) % 4294967296; return seed / 4294967296; };
    const tokens = words.map((w, i) => ({ original_index: i, id: 100 + i, piece: w.replace(' ', 'Ġ'),
      display: w.replace(' ', '·'), source: i < prompt ? 'prompt' : 'generated' }));
    const labels = tokens.map((t) => t.original_index + ':' + t.display);
    const cols = [];
    for (let b = 0; b < bins; b++) cols.push((8 * b) + '..' + (8 * b + 7));
    const heat = (rows, ncols, rl, cl, f, kind) => {
      const values = [];
      for (let r = 0; r < rows; r++) for (let c = 0; c < ncols; c++) values.push(f(r, c));
      return { rows, cols: ncols, row_labels: rl, col_labels: cl, values, min: Math.min(...values), max: Math.max(...values),
        value_kind: kind, original_rows: rows, original_cols: kind === 'signed_mean' ? 256 : ncols };
    };
    const stage = (name, label, i, mixer) => {
      const s = { stage: name, label };
      if (i !== null) { s.layer_index = i + 1; s.mixer = mixer; }
      const d = i === null ? 0 : i + 1;
      s.activation = heat(n, bins, labels, cols, (t, b) => Math.sin(0.3 * b + 0.5 * d + 0.2 * t) * (0.4 + rnd()), 'signed_mean');
      s.stats = { mean: 0, rms: 1 + 0.35 * d, min: s.activation.min, max: s.activation.max,
        abs_max: Math.max(Math.abs(s.activation.min), Math.abs(s.activation.max)) };
      s.token_rms = tokens.map(() => 1 + 0.35 * d + 0.2 * rnd());
      if (name !== 'embedding') s.token_delta_rms = tokens.map(() => 0.2 + 0.1 * rnd());
      return s;
    };
    const stages = [stage('embedding', 'Token embedding', null, null)];
    const arch = [];
    for (let i = 0; i < L; i++) {
      const mamba = i === 2;
      const s = stage('block', 'Layer ' + (i + 1) + ' · ' + (mamba ? 'mamba' : 'attention'), i, mamba ? 'mamba' : 'attention');
      if (mamba) {
        s.mamba_state = heat(16, bins, Array.from({ length: 16 }, (_, j) => 'state ' + j), cols,
          (r, c) => Math.cos(0.4 * r + 0.2 * c) * rnd(), 'signed_mean');
      } else {
        const heads = [];
        for (let h = 0; h < 2; h++) {
          const rowsum = new Array(n).fill(0), raw = [];
          for (let q = 0; q < n; q++) for (let k = 0; k < n; k++) {
            const v = k <= q ? Math.exp(-Math.abs(q - k - h * (i % 3)) / (1 + h + 0.5 * i)) + 0.05 * rnd() : 0;
            raw.push(v); rowsum[q] += v;
          }
          heads.push(heat(n, n, labels, labels, (q, k) => raw[q * n + k] / rowsum[q], 'probability'));
        }
        s.attention = { total_heads: 4, captured_heads: 2, heads };
      }
      stages.push(s);
      arch.push({ index: i + 1, name: mamba ? 'm' : 'a', mixer: mamba
        ? { kind: 'mamba', state_dim: 16, conv_kernel: 4, expand: 2, dt_rank: 16, inner_size: 512 }
        : { kind: 'attention', num_heads: 4, num_kv_heads: 4, head_dim: 64, causal: true, qk_norm: false, position_encoding: 'rope' },
        ffn_hidden_size: 1024, ffn_activation: 'swiglu', ffn_gated: true, norm: 'rmsnorm', norm_position: 'pre',
        residual: true, dropout: 0 });
    }
    stages.push(stage('final_norm', 'Final norm', null, null));
    const rows = [];
    for (let s = 1; s <= 60; s++) {
      rows.push({ schema_version: 2, sequence: 2 * s - 2, global_step: s, event: { type: 'optimization',
        values: { loss: 5.5 * Math.exp(-s / 25) + 2 + 0.1 * rnd(), gradient_norm: 1.5 * Math.exp(-s / 40) + 0.3 * rnd(), learning_rate: 3e-4 * Math.min(1, s / 10) } } });
      rows.push({ schema_version: 2, sequence: 2 * s - 1, global_step: s, event: { type: 'throughput',
        values: { tokens_per_second: 250000 + 20000 * rnd(), elapsed_seconds: 0.06 } } });
    }
    return {
      kind: 'summa_model_trace', version: 1,
      model: { name: 'demo', vocab_size: 32000, max_seq_len: 2048, hidden_size: 256, num_layers: L,
        estimated_parameters: 12500000, tied_embeddings: true, layers: arch },
      inference: { prompt: words.slice(0, prompt).join(''), generated_text: words.slice(prompt).join(''),
        full_text: words.join(''), original_token_count: n, prompt_token_count: prompt, generated_token_count: n - prompt,
        token_offset: 0, tokens,
        sampling: { max_new_tokens: 3, temperature: 0, repetition_penalty: 1, seed: 0, stop_at_eos: true }, stages },
      training: { source: 'demo', total_rows: rows.length, captured_rows: rows.length, dropped_rows: 0, sampling_stride: 1, rows },
      capture: { requested_token_limit: 128, original_tokens: n, captured_tokens: n, dropped_leading_tokens: 0,
        tokens_truncated: false, original_hidden_channels: 256, captured_hidden_channels: bins, channels_reduced: true,
        requested_attention_head_limit: 2, metrics_total_rows: rows.length, metrics_captured_rows: rows.length },
    };
  }
  if (typeof module !== 'undefined' && module.exports) module.exports = { makeDemoTrace };
  else root.makeDemoTrace = makeDemoTrace;
})(typeof window !== 'undefined' ? window : globalThis);
