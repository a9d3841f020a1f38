// Control block and ring record shared by the device kernels and the host runtime.
//
// The control block is 16 int32 words in device memory; every kernel of a round reads its inputs
// (positions, counters) from it and the tail kernel is the only writer during decoding.
// Reference counterpart: naivert/runtime/mtp_contract.py (_DecodeControlLayout, 80 bytes) and
// naivert/runtime/sequencer.py (_SequencerOutputRecordLayout, 48 bytes).
#pragma once

enum NrtCtrl : int {
  NRT_CTRL_POS = 0,          // position of row 0 of the next step (= rows valid in the caches)
  NRT_CTRL_COMMITTED = 1,    // tokens committed by the last round (feature rows the next ingest may use)
  NRT_CTRL_INGEST_POS = 2,   // first position of the next draft ingest
  NRT_CTRL_RESERVED3 = 3,
  NRT_CTRL_STOPPED = 4,      // non-zero once the request has stopped; later rounds publish nothing
  NRT_CTRL_REASON = 5,       // stop reason (see NrtStop)
  NRT_CTRL_GENERATED = 6,    // tokens generated so far
  NRT_CTRL_MAX_TOKENS = 7,
  NRT_CTRL_ROUND = 8,        // round counter (Philox counter, ring generation)
  NRT_CTRL_CAPACITY = 9,     // cache capacity in positions
  NRT_CTRL_CURSOR = 10,      // prompt replay cursor
  NRT_CTRL_PROMPT_CTX = 11,  // prompt context length (prompt tokens - 1)
  NRT_CTRL_RELAUNCH_FAIL = 12,   // device-side relaunch failures
  NRT_CTRL_PAUSED = 13,      // the device chain paused for host backpressure
  NRT_CTRL_WORDS = 16
};

enum NrtStop : int {
  NRT_STOP_NONE = 0,
  NRT_STOP_EOS = 1,
  NRT_STOP_MAX_TOKENS = 2,
  NRT_STOP_CAPACITY = 3,
  NRT_STOP_CANCELLED = 4,
  NRT_STOP_DEVICE_WAIT_FAILED = 5,
  NRT_STOP_RELAUNCH_FAILED = 6
};
