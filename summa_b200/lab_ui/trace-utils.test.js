// node summa_b200/lab_ui/trace-utils.test.js
const assert = require('assert');
const U = require('./trace-utils.js');
const { makeDemoTrace } = require('./demo-trace.js');

const t = makeDemoTrace();
assert.strictEqual(U.validateTrace(t), t);
assert.strictEqual(U.parseTraceJson(JSON.stringify(t)).tokens.length, 12);
assert.throws(() => U.parseTraceJson('{'), /not JSON/);
assert.throws(() => U.validateTrace({ ...t, format: 'other' }), /format/);
assert.throws(() => U.validateTrace({ ...t, version: 2 }), /version/);
assert.throws(() => U.validateTrace({ ...t, tokens: [] }), /token count/);
const bad = JSON.parse(JSON.stringify(t));
bad.layers[0].attention[0][3] = [1, 2];
assert.throws(() => U.validateTrace(bad), /head 0 shape/);

const r = U.resample([[0, 1], [2, 3]], 3, 3);
assert.deepStrictEqual(r[1], [1, 1.5, 2]);
assert.deepStrictEqual(U.extent([[2, 2]]), [2, 3]);
assert.deepStrictEqual(U.colour(0), [13, 8, 135]);
assert.deepStrictEqual(U.colour(1), [253, 231, 37]);
const s = U.metricSeries(t.metrics);
assert.strictEqual(s.loss.length, 60);
assert.ok(s.tokens_per_second[0][1] > 0);
assert.strictEqual(U.layerNormProfile(t).length, 6);
console.log('trace-utils: ok');
