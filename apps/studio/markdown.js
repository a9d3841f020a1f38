// A deliberately small Markdown renderer for model output: fenced code, inline code, bold, italics, headings,
// unordered lists, paragraphs.  Everything is escaped first; no raw HTML from the model reaches the page.
const ESC = { "&": "&amp;", "<": "&lt;", ">": "&gt;", '"': "&quot;", "'": "&#39;" };
export const escapeHtml = (s) => s.replace(/[&<>"']/g, (c) => ESC[c]);
function inline(s) {
  return s.replace(/`([^`]+)`/g, "<code>$1</code>")
          .replace(/\*\*([^*]+)\*\*/g, "<strong>$1</strong>")
          .replace(/(^|[^*])\*([^*\s][^*]*)\*/g, "$1<em>$2</em>");
}
export function renderMarkdown(text) {
  const out = [];
  const lines = escapeHtml(text).split("\n");
  let i = 0, list = false, para = [];
  const flushPara = () => { if (para.length) { out.push(`<p>${inline(para.join(" "))}</p>`); para = []; } };
  const closeList = () => { if (list) { out.push("</ul>"); list = false; } };
  while (i < lines.length) {
    const line = lines[i];
    if (line.startsWith("```")) {
      flushPara(); closeList();
      const lang = line.slice(3).trim();
      const body = [];
      for (i++; i < lines.length && !lines[i].startsWith("```"); i++) body.push(lines[i]);
      out.push(`<pre><code${lang ? ` class="language-${lang.replace(/[^\w-]/g, "")}"` : ""}>${body.join("\n")}</code></pre>`);
      i++;                                         // closing fence (or end of text: an unterminated block still renders)
      continue;
    }
    const h = /^(#{1,4})\s+(.*)$/.exec(line);
    if (h) { flushPara(); closeList(); out.push(`<h${h[1].length}>${inline(h[2])}</h${h[1].length}>`); }
    else if (/^\s*[-*]\s+/.test(line)) { flushPara(); if (!list) { out.push("<ul>"); list = true; } out.push(`<li>${inline(line.replace(/^\s*[-*]\s+/, ""))}</li>`); }
    else if (line.trim() === "") { flushPara(); closeList(); }
    else { closeList(); para.push(line.trim()); }
    i++;
  }
  flushPara(); closeList();
  return out.join("\n");
}
