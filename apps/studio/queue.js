// Request queue of the Studio client: the server runs one sequence at a time, so prompts typed while a request is
// running wait here in order.  Pure logic (no DOM): the page subscribes with onChange.
export class RequestQueue {
  constructor(runner) {
    this.runner = runner;          // async (item) => result; the queue awaits it before starting the next item
    this.items = [];               // waiting items, oldest first
    this.active = null;
    this.nextId = 1;
    this.listeners = [];
  }
  onChange(fn) { this.listeners.push(fn); }
  _emit() { for (const fn of this.listeners) fn(this.snapshot()); }
  snapshot() { return { active: this.active, waiting: this.items.map((i) => ({ id: i.id, prompt: i.prompt })) }; }
  push(prompt, options = {}) {
    const item = { id: this.nextId++, prompt, options, state: "waiting" };
    this.items.push(item);
    this._emit();
    this._pump();
    return item.id;
  }
  remove(id) {                     // a waiting item can be withdrawn; the active one is cancelled through its AbortController
    const n = this.items.length;
    this.items = this.items.filter((i) => i.id !== id);
    if (this.items.length !== n) this._emit();
    return this.items.length !== n;
  }
  clear() { this.items = []; this._emit(); }
  async _pump() {
    if (this.active || this.items.length === 0) return;
    const item = this.items.shift();
    this.active = { id: item.id, prompt: item.prompt };
    item.state = "running";
    this._emit();
    try { item.result = await this.runner(item); item.state = "done"; }
    catch (e) { item.error = e; item.state = "failed"; }
    this.active = null;
    this._emit();
    this._pump();
  }
}
