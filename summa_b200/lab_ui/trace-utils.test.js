// node summa_b200/lab_ui/trace-utils.test.js
const assert = require('assert');
const U = require('./trace-utils.js');
const { makeDemoTrace } = require('./demo-trace.js');

const t = makeDemoTrace();
const view = U.validateTrace(t);
assert.strictEqual(view.bundle, t);
assert.strictEqual(view.tokens.length, 12);
assert.strictEqual(view.layers.length, 6);
assert.strictEqual(view.layers[2].mixer, 'mamba');
assert.strictEqual(view.layers[2].mamba_state.length, 16);
assert.strictEqual(view.layers[0].attention[0].length, 12);
assert.strictEqual(U.parseTraceJson(JSON.stringify(t)).tokens.length, 12);
assert.throws(() => U.parseTraceJson('{'), /not JSON/);
assert.throws(() => U.validateTrace({ ...t, kind: 'other' }), /kind/);
assert.throws(() => U.validateTrace({ ...t, version: 2 }), /version/);
assert.throws(() => U.validateTrace({ ...t, inference: { ...t.inference, tokens: [] } }), /token count/);
const bad = JSON.parse(JSON.stringify(t));
bad.inference.stages[1].attention.heads[0].values.pop();
assert.throws(() => U.validateTrace(bad), /head 0 heat-map values/);

const r = U.resample([[0, 1], [2, 3]], 3, 3);
assert.deepStrictEqual(r[1], [1, 1.5, 2]);
assert.deepStrictEqual(U.extent([[2, 2]]), [2, 3]);
assert.deepStrictEqual(U.colour(0), [13, 8, 135]);
assert.deepStrictEqual(U.colour(1), [253, 231, 37]);
const s = U.metricSeries(view.metrics);
assert.strictEqual(s.loss.length, 60);
assert.ok(s.tokens_per_second[0][1] > 0);
assert.strictEqual(U.layerNormProfile(view).length, 6);
console.log('trace-utils: ok');
