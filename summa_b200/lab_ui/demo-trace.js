// A synthetic trace (no model needed): 12 tokens through a 6-block stack with one state-space
// block, banded causal attention patterns and a decaying loss curve.
(function (root) {
  'use strict';
  function makeDemoTrace() {
    const words = ['The', ' quick', ' brown', ' fox', ' jumps', ' over', ' the', ' lazy', ' dog', ' and', ' runs', ' away'];
    const n = words.length, layers = [];
    let seed = 7;
    const rnd = () => { seed = (seed * 1664525 + 1013904223) % 4294967296; return seed / 4294967296; };
    for (let i = 0; i < 6; i++) {
      const l = { index: i, mixer: i === 2 ? 'ssm' : 'attention', residual_norm: [], channels: [] };
      for (let t = 0; t < n; t++) {
        l.residual_norm.push(1 + 0.35 * i + 0.2 * rnd());
        const bins = [];
        for (let b = 0; b < 32; b++) bins.push(Math.abs(Math.sin(0.3 * b + 0.5 * i + 0.2 * t)) * (0.4 + rnd()));
        l.channels.push(bins);
      }
      if (l.mixer === 'attention') {
        l.attention = [];
        for (let h = 0; h < 2; h++) {
          const head = [];
          for (let q = 0; q < n; q++) {
            const row = new Array(n).fill(0);
            let sum = 0;
            for (let k = 0; k <= q; k++) { row[k] = Math.exp(-Math.abs(q - k - h * (i % 3)) / (1 + h + 0.5 * i)) + 0.05 * rnd(); sum += row[k]; }
            for (let k = 0; k <= q; k++) row[k] /= sum;
            head.push(row);
          }
          l.attention.push(head);
        }
      }
      layers.push(l);
    }
    const metrics = [];
    for (let s = 1; s <= 60; s++) {
      metrics.push({ schema_version: 2, sequence: 2 * s, global_step: s, event: { type: 'optimization',
        values: { loss: 5.5 * Math.exp(-s / 25) + 2 + 0.1 * rnd(), gradient_norm: 1.5 * Math.exp(-s / 40) + 0.3 * rnd(), learning_rate: 3e-4 * Math.min(1, s / 10) } } });
      metrics.push({ schema_version: 2, sequence: 2 * s + 1, global_step: s, event: { type: 'throughput',
        values: { tokens_per_second: 250000 + 20000 * rnd(), elapsed_seconds: 0.06 } } });
    }
    return {
      format: 'summa_model_trace', version: 1,
      model: { name: 'demo', hidden_size: 256, num_layers: 6, vocab_size: 32000, parameters: 12.5e6 },
      tokens: words.map((w, i) => ({ id: 100 + i, text: w })),
      layers,
      next_token: [{ id: 7, text: '.', probability: 0.41 }, { id: 8, text: ' quickly', probability: 0.22 },
        { id: 9, text: ' again', probability: 0.12 }, { id: 10, text: ',', probability: 0.08 }],
      metrics,
    };
  }
  if (typeof module !== 'undefined' && module.exports) module.exports = { makeDemoTrace };
  else root.makeDemoTrace = makeDemoTrace;
})(typeof window !== 'undefined' ? window : globalThis);
