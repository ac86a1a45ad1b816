// Result dump formats: JSON, CSV and XML writers whose output is
// byte-compatible with the reference's (src/common/result_store.cpp:149-448,
// format_version 2), and loaders for all three.
//
// The loaders here are small real parsers rather than line scanners: the XML
// one walks elements and attributes wherever the line breaks fall, the JSON
// one walks objects inside the "devices" and "entries" arrays.  They accept
// everything the writers produce and ignore keys / attributes they do not know,
// which is what lets newer files load in older builds and vice versa.
#include <cstring>
#include <fstream>
#include <iomanip>
#include <locale>
#include <sstream>

#include "clpeak_api.hpp"

namespace {

// ---- number formatting: always the classic locale -----------------------------

std::string fixed4(float v)
{
    std::ostringstream ss;
    ss.imbue(std::locale::classic());
    ss << std::fixed << std::setprecision(4) << v;
    return ss.str();
}

bool parseFloatClassic(const std::string &text, float &out)
{
    std::istringstream is(text);
    is.imbue(std::locale::classic());
    float v = 0.0f;
    if (!(is >> v))
        return false;
    out = v;
    return true;
}

std::string csvQuote(const std::string &s)
{
    std::string out = "\"";
    for (char c : s) {
        if (c == '"')
            out += "\"\"";
        else
            out += c;
    }
    out += "\"";
    return out;
}

std::string xmlEscape(const std::string &s)
{
    std::string out;
    out.reserve(s.size() + 16);
    for (char c : s) {
        switch (c) {
        case '&': out += "&amp;"; break;
        case '<': out += "&lt;"; break;
        case '>': out += "&gt;"; break;
        case '\'': out += "&apos;"; break;
        case '"': out += "&quot;"; break;
        default: out += c;
        }
    }
    return out;
}

std::string xmlUnescape(const std::string &s)
{
    static const struct { const char *ent; char ch; } kEnt[] = {
        {"&amp;", '&'}, {"&lt;", '<'}, {"&gt;", '>'}, {"&apos;", '\''}, {"&quot;", '"'}};
    std::string out;
    out.reserve(s.size());
    for (size_t i = 0; i < s.size();) {
        bool hit = false;
        if (s[i] == '&') {
            for (const auto &e : kEnt) {
                const size_t n = std::strlen(e.ent);
                if (s.compare(i, n, e.ent) == 0) {
                    out += e.ch;
                    i += n;
                    hit = true;
                    break;
                }
            }
        }
        if (!hit)
            out += s[i++];
    }
    return out;
}

bool versionAccepted(int got, const std::string &file)
{
    if (got == RESULT_FORMAT_VERSION)
        return true;
    std::cerr << "clpeak: " << file << " is format_version=" << got << "; this build expects v"
              << RESULT_FORMAT_VERSION << ". Regenerate the file with this version of clpeak.\n";
    return false;
}

void writeJsonDoc(const ResultStore &store, const DeviceInfoStore &devices, std::ostream &f)
{
    f.imbue(std::locale::classic());
    f << "{\"format_version\":" << RESULT_FORMAT_VERSION << ",\"clpeak_version\":\""
      << jsonEscape(CLPEAK_VERSION_STR) << "\",\"os\":\"" << jsonEscape(OS_NAME) << "\"";
    if (!devices.empty()) {
        f << ",\"devices\":[\n";
        for (size_t i = 0; i < devices.size(); ++i) {
            const DeviceInfo &d = devices[i];
            f << "{\"backend\":\"" << jsonEscape(d.backend) << "\",\"platform\":\"" << jsonEscape(d.platform)
              << "\",\"device\":\"" << jsonEscape(d.device) << "\",\"driver\":\"" << jsonEscape(d.driver)
              << "\",\"props\":[";
            for (size_t j = 0; j < d.props.size(); ++j)
                f << (j ? "," : "") << "{\"k\":\"" << jsonEscape(d.props[j].key) << "\",\"v\":\""
                  << jsonEscape(d.props[j].value) << "\"}";
            f << "]}" << (i + 1 < devices.size() ? "," : "") << "\n";
        }
        f << "]";
    }
    f << ",\"entries\":[\n";
    for (size_t i = 0; i < store.size(); ++i) {
        const ResultEntry &e = store[i];
        f << "{\"backend\":\"" << jsonEscape(e.backend) << "\",\"platform\":\"" << jsonEscape(e.platform)
          << "\",\"device\":\"" << jsonEscape(e.device) << "\",\"driver\":\"" << jsonEscape(e.driver)
          << "\",\"category\":\"" << jsonEscape(e.category) << "\",\"test\":\"" << jsonEscape(e.test)
          << "\",\"metric\":\"" << jsonEscape(e.metric) << "\",\"unit\":\"" << jsonEscape(e.unit) << "\"";
        if (!e.display.empty())
            f << ",\"display\":\"" << jsonEscape(e.display) << "\"";
        if (!e.description.empty())
            f << ",\"description\":\"" << jsonEscape(e.description) << "\"";
        if (!e.metricDescription.empty())
            f << ",\"metric_description\":\"" << jsonEscape(e.metricDescription) << "\"";
        if (e.status == ResultStatus::Ok)
            f << ",\"value\":" << fixed4(e.value);
        else
            f << ",\"status\":\"" << statusString(e.status) << "\",\"reason\":\"" << jsonEscape(e.reason) << "\"";
        f << "}" << (i + 1 < store.size() ? "," : "") << "\n";
    }
    f << "]}\n";
}

// ---- a minimal JSON value walker ---------------------------------------------------
// Enough for the documents above: objects, arrays, strings with escapes,
// numbers, true/false/null.  Objects are returned as flat key -> raw-value maps
// with string values already unescaped; nested containers keep their raw text.

struct JsonCursor {
    const std::string &s;
    size_t i = 0;
    explicit JsonCursor(const std::string &text) : s(text) {}

    void ws()
    {
        while (i < s.size() && std::isspace((unsigned char)s[i]))
            ++i;
    }
    bool eat(char c)
    {
        ws();
        if (i < s.size() && s[i] == c) {
            ++i;
            return true;
        }
        return false;
    }
    bool string(std::string &out)
    {
        ws();
        if (i >= s.size() || s[i] != '"')
            return false;
        ++i;
        out.clear();
        while (i < s.size() && s[i] != '"') {
            char c = s[i++];
            if (c == '\\' && i < s.size()) {
                char n = s[i++];
                switch (n) {
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u':
                    if (i + 4 <= s.size()) {
                        out += (char)std::strtol(s.substr(i, 4).c_str(), nullptr, 16);
                        i += 4;
                    }
                    break;
                default: out += n;
                }
            } else {
                out += c;
            }
        }
        if (i >= s.size())
            return false;
        ++i;
        return true;
    }
    // Skips one value of any type and returns its raw text.
    bool raw(std::string &out)
    {
        ws();
        const size_t start = i;
        if (i >= s.size())
            return false;
        if (s[i] == '"') {
            std::string tmp;
            if (!string(tmp))
                return false;
        } else if (s[i] == '{' || s[i] == '[') {
            int depth = 0;
            bool inStr = false;
            for (; i < s.size(); ++i) {
                char c = s[i];
                if (inStr) {
                    if (c == '\\')
                        ++i;
                    else if (c == '"')
                        inStr = false;
                } else if (c == '"') {
                    inStr = true;
                } else if (c == '{' || c == '[') {
                    ++depth;
                } else if (c == '}' || c == ']') {
                    if (--depth == 0) {
                        ++i;
                        break;
                    }
                }
            }
        } else {
            while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']' && !std::isspace((unsigned char)s[i]))
                ++i;
        }
        out = s.substr(start, i - start);
        return i > start;
    }
};

using FlatObject = std::map<std::string, std::string>;     // key -> value (strings unescaped, rest raw)

bool parseFlatObject(JsonCursor &c, FlatObject &obj)
{
    obj.clear();
    if (!c.eat('{'))
        return false;
    if (c.eat('}'))
        return true;
    do {
        std::string key;
        if (!c.string(key) || !c.eat(':'))
            return false;
        c.ws();
        std::string val;
        if (c.i < c.s.size() && c.s[c.i] == '"') {
            if (!c.string(val))
                return false;
            obj[key] = val;
            obj["\x01" + key] = "s";                         // marks "was a string"
        } else {
            if (!c.raw(val))
                return false;
            obj[key] = val;
        }
    } while (c.eat(','));
    return c.eat('}');
}

template <typename Fn>
bool forEachObjectInArray(const std::string &rawArray, Fn fn)
{
    JsonCursor c(rawArray);
    if (!c.eat('['))
        return false;
    if (c.eat(']'))
        return true;
    do {
        FlatObject o;
        if (!parseFlatObject(c, o))
            return false;
        fn(o);
    } while (c.eat(','));
    return c.eat(']');
}

std::string get(const FlatObject &o, const char *k)
{
    auto it = o.find(k);
    return it == o.end() ? std::string() : it->second;
}

bool rowComplete(const ResultEntry &e) { return !e.backend.empty() && !e.test.empty() && !e.metric.empty(); }

std::string slurp(const std::string &filename, bool &ok)
{
    std::ifstream f(filename, std::ios::binary);
    ok = f.is_open();
    if (!ok) {
        std::cerr << "clpeak: cannot open compare file: " << filename << "\n";
        return {};
    }
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

void warnEmpty(const ResultStore &st, const std::string &filename)
{
    if (st.empty())
        std::cerr << "clpeak: warning: no valid entries found in: " << filename << "\n";
}

} // namespace

// ===========================================================================
// Writers
// ===========================================================================

bool saveJson(const ResultStore &store, const std::string &filename, const DeviceInfoStore &devices)
{
    std::ofstream f(filename);
    if (!f.is_open()) {
        std::cerr << "clpeak: cannot open JSON output file: " << filename << "\n";
        return false;
    }
    writeJsonDoc(store, devices, f);
    return f.good();
}

std::string resultsToJson(const ResultStore &store, const DeviceInfoStore &devices)
{
    std::ostringstream ss;
    writeJsonDoc(store, devices, ss);
    return ss.str();
}

bool saveCsv(const ResultStore &store, const std::string &filename)
{
    std::ofstream f(filename);
    if (!f.is_open()) {
        std::cerr << "clpeak: cannot open CSV output file: " << filename << "\n";
        return false;
    }
    f.imbue(std::locale::classic());
    f << "format_version,backend,platform,device,driver,category,test,metric,unit,status,value,reason,display,"
         "description,metric_description\n";
    for (const ResultEntry &e : store) {
        const std::string cells[] = {e.backend, e.platform, e.device, e.driver, e.category,
                                     e.test,    e.metric,   e.unit,   statusString(e.status)};
        f << RESULT_FORMAT_VERSION;
        for (const std::string &c : cells)
            f << "," << csvQuote(c);
        f << "," << (e.status == ResultStatus::Ok ? fixed4(e.value) : std::string());
        f << "," << csvQuote(e.reason) << "," << csvQuote(e.display) << "," << csvQuote(e.description) << ","
          << csvQuote(e.metricDescription) << "\n";
    }
    return f.good();
}

// One linear pass; rows arrive grouped run -> category -> test because backends
// emit them in run order.  An element is closed when the next row leaves it.
bool saveXml(const ResultStore &store, const std::string &filename, const DeviceInfoStore &devices)
{
    std::ofstream f(filename);
    if (!f.is_open()) {
        std::cerr << "clpeak: cannot open XML output file: " << filename << "\n";
        return false;
    }
    f.imbue(std::locale::classic());
    f << "<?xml version=\"1.0\" encoding=\"utf-8\"?>\n"
      << "<clpeak format_version=\"" << RESULT_FORMAT_VERSION << "\" clpeak_version=\""
      << xmlEscape(CLPEAK_VERSION_STR) << "\" os=\"" << xmlEscape(OS_NAME) << "\">\n";

    enum Level { None = 0, Run = 1, Cat = 2, Test = 3 };
    int open = None;
    std::string runKey, cat, test, unit;
    auto closeTo = [&](int level) {
        if (open >= Test && level < Test) f << "      </test>\n";
        if (open >= Cat && level < Cat) f << "    </category>\n";
        if (open >= Run && level < Run) f << "  </run>\n";
        open = std::min(open, level);
    };

    for (const ResultEntry &e : store) {
        const std::string key = e.backend + "/" + e.platform + "/" + e.device + "/" + e.driver;
        if (open < Run || key != runKey) {
            closeTo(None);
            f << "  <run backend=\"" << xmlEscape(e.backend) << "\" platform=\"" << xmlEscape(e.platform)
              << "\" device=\"" << xmlEscape(e.device) << "\" driver=\"" << xmlEscape(e.driver) << "\">\n";
            for (const DeviceInfo &d : devices) {
                if (d.key() != key)
                    continue;
                for (const DeviceProp &p : d.props)
                    f << "    <prop name=\"" << xmlEscape(p.key) << "\" value=\"" << xmlEscape(p.value) << "\"/>\n";
                break;
            }
            open = Run;
            runKey = key;
        }
        if (open < Cat || cat != e.category) {
            closeTo(Run);
            f << "    <category name=\"" << xmlEscape(e.category) << "\">\n";
            open = Cat;
            cat = e.category;
        }
        if (open < Test || test != e.test || unit != e.unit) {
            closeTo(Cat);
            f << "      <test name=\"" << xmlEscape(e.test) << "\"";
            if (!e.display.empty())
                f << " display=\"" << xmlEscape(e.display) << "\"";
            f << " unit=\"" << xmlEscape(e.unit) << "\"";
            if (!e.description.empty())
                f << " description=\"" << xmlEscape(e.description) << "\"";
            f << ">\n";
            open = Test;
            test = e.test;
            unit = e.unit;
        }
        f << "        <metric name=\"" << xmlEscape(e.metric) << "\"";
        if (!e.metricDescription.empty())
            f << " info=\"" << xmlEscape(e.metricDescription) << "\"";
        if (e.status == ResultStatus::Ok)
            f << ">" << fixed4(e.value) << "</metric>\n";
        else
            f << " status=\"" << statusString(e.status) << "\" reason=\"" << xmlEscape(e.reason) << "\"/>\n";
    }
    closeTo(None);
    f << "</clpeak>\n";
    return f.good();
}

// ===========================================================================
// Loaders
// ===========================================================================

ResultStore loadJson(const std::string &filename, DeviceInfoStore *devices)
{
    ResultStore store;
    bool ok = false;
    const std::string text = slurp(filename, ok);
    if (!ok)
        return store;

    JsonCursor c(text);
    c.ws();
    if (c.i >= text.size() || text[c.i] != '{') {
        versionAccepted(1, filename);          // bare array or garbage: unversioned
        return store;
    }
    // top-level object: keep containers raw
    FlatObject top;
    if (!parseFlatObject(c, top) || top.find("format_version") == top.end()) {
        versionAccepted(1, filename);
        return store;
    }
    if (!versionAccepted(std::atoi(top["format_version"].c_str()), filename))
        return store;

    if (devices && top.count("devices")) {
        forEachObjectInArray(top["devices"], [&](const FlatObject &o) {
            DeviceInfo d;
            d.backend = get(o, "backend");
            d.platform = get(o, "platform");
            d.device = get(o, "device");
            d.driver = get(o, "driver");
            forEachObjectInArray(get(o, "props"), [&](const FlatObject &p) {
                DeviceProp prop{get(p, "k"), get(p, "v")};
                if (!prop.key.empty())
                    d.props.push_back(prop);
            });
            if (!d.backend.empty())
                devices->push_back(d);
        });
    }
    if (top.count("entries")) {
        forEachObjectInArray(top["entries"], [&](const FlatObject &o) {
            ResultEntry e;
            e.backend = get(o, "backend");
            e.platform = get(o, "platform");
            e.device = get(o, "device");
            e.driver = get(o, "driver");
            e.category = get(o, "category");
            e.test = get(o, "test");
            e.metric = get(o, "metric");
            e.unit = get(o, "unit");
            e.display = get(o, "display");
            e.description = get(o, "description");
            e.metricDescription = get(o, "metric_description");
            if (o.count("status")) {
                e.status = statusFromString(get(o, "status"));
                e.reason = get(o, "reason");
            } else {
                e.status = ResultStatus::Ok;
                parseFloatClassic(get(o, "value"), e.value);
            }
            if (rowComplete(e))
                store.push_back(e);
        });
    }
    warnEmpty(store, filename);
    return store;
}

ResultStore loadCsv(const std::string &filename)
{
    ResultStore store;
    std::ifstream f(filename);
    if (!f.is_open()) {
        std::cerr << "clpeak: cannot open compare file: " << filename << "\n";
        return store;
    }
    auto split = [](const std::string &line, std::vector<std::string> &cells) {
        cells.clear();
        std::string cur;
        bool quoted = false;
        for (size_t i = 0; i < line.size(); ++i) {
            const char ch = line[i];
            if (quoted) {
                if (ch != '"')
                    cur += ch;
                else if (i + 1 < line.size() && line[i + 1] == '"')
                    cur += '"', ++i;
                else
                    quoted = false;
            } else if (ch == '"') {
                quoted = true;
            } else if (ch == ',') {
                cells.push_back(cur);
                cur.clear();
            } else if (ch != '\r') {
                cur += ch;
            }
        }
        cells.push_back(cur);
        return !quoted;
    };

    std::string line;
    std::getline(f, line);                    // header
    bool versionSeen = false;
    std::vector<std::string> c;
    while (std::getline(f, line)) {
        if (line.empty() || line[0] == '\r')
            continue;
        if (!split(line, c)) {
            std::cerr << "clpeak: warning: skipping malformed CSV line in: " << filename << "\n";
            continue;
        }
        if (c.size() < 12) {
            if (!versionSeen) {
                versionAccepted(1, filename);
                return store;
            }
            continue;
        }
        if (!versionSeen) {
            if (!versionAccepted(std::atoi(c[0].c_str()), filename))
                return store;
            versionSeen = true;
        }
        ResultEntry e;
        e.backend = c[1];
        e.platform = c[2];
        e.device = c[3];
        e.driver = c[4];
        e.category = c[5];
        e.test = c[6];
        e.metric = c[7];
        e.unit = c[8];
        e.status = statusFromString(c[9]);
        if (e.status == ResultStatus::Ok && !parseFloatClassic(c[10], e.value))
            continue;
        e.reason = c[11];
        if (c.size() > 12) e.display = c[12];
        if (c.size() > 13) e.description = c[13];
        if (c.size() > 14) e.metricDescription = c[14];
        if (rowComplete(e))
            store.push_back(e);
    }
    warnEmpty(store, filename);
    return store;
}

namespace {

// One start tag (or empty-element tag) with its attributes, plus the text that
// follows it up to the next '<'.
struct XmlTag {
    std::string name;
    std::map<std::string, std::string> attr;
    std::string text;
    bool closing = false;
};

bool nextTag(const std::string &s, size_t &pos, XmlTag &tag)
{
    tag = XmlTag();
    size_t lt = s.find('<', pos);
    if (lt == std::string::npos)
        return false;
    size_t gt = lt + 1;
    bool inQuote = false;
    for (; gt < s.size(); ++gt) {
        if (s[gt] == '"')
            inQuote = !inQuote;
        else if (s[gt] == '>' && !inQuote)
            break;
    }
    if (gt >= s.size())
        return false;
    std::string body = s.substr(lt + 1, gt - lt - 1);
    pos = gt + 1;
    if (!body.empty() && (body[0] == '?' || body[0] == '!')) {
        tag.name = "?";
        return true;
    }
    if (!body.empty() && body[0] == '/') {
        tag.closing = true;
        tag.name = body.substr(1);
        return true;
    }
    if (!body.empty() && body.back() == '/')
        body.pop_back();
    size_t i = 0;
    while (i < body.size() && !std::isspace((unsigned char)body[i]))
        ++i;
    tag.name = body.substr(0, i);
    while (i < body.size()) {
        while (i < body.size() && std::isspace((unsigned char)body[i]))
            ++i;
        size_t eq = body.find('=', i);
        if (eq == std::string::npos)
            break;
        std::string key = body.substr(i, eq - i);
        size_t q1 = body.find('"', eq);
        if (q1 == std::string::npos)
            break;
        size_t q2 = body.find('"', q1 + 1);
        if (q2 == std::string::npos)
            break;
        tag.attr[key] = xmlUnescape(body.substr(q1 + 1, q2 - q1 - 1));
        i = q2 + 1;
    }
    size_t nextLt = s.find('<', pos);
    tag.text = s.substr(pos, (nextLt == std::string::npos ? s.size() : nextLt) - pos);
    return true;
}

} // namespace

ResultStore loadXml(const std::string &filename, DeviceInfoStore *devices)
{
    ResultStore store;
    bool ok = false;
    const std::string text = slurp(filename, ok);
    if (!ok)
        return store;

    size_t pos = 0;
    XmlTag t;
    bool versionSeen = false;
    ResultEntry ctx;                 // run / category / test context for the rows below
    DeviceInfo dev;
    auto flushDevice = [&]() {
        if (devices && !dev.props.empty())
            devices->push_back(dev);
        dev = DeviceInfo();
    };
    while (nextTag(text, pos, t)) {
        if (t.closing || t.name == "?")
            continue;
        if (t.name == "clpeak") {
            if (!versionAccepted(std::atoi(t.attr["format_version"].c_str()), filename))
                return store;
            versionSeen = true;
            continue;
        }
        if (!versionSeen) {
            versionAccepted(0, filename);
            return store;
        }
        if (t.name == "run") {
            flushDevice();
            ctx = ResultEntry();
            ctx.backend = dev.backend = t.attr["backend"];
            ctx.platform = dev.platform = t.attr["platform"];
            ctx.device = dev.device = t.attr["device"];
            ctx.driver = dev.driver = t.attr["driver"];
        } else if (t.name == "prop") {
            if (!t.attr["name"].empty())
                dev.props.push_back({t.attr["name"], t.attr["value"]});
        } else if (t.name == "category") {
            ctx.category = t.attr["name"];
            ctx.test.clear();
            ctx.unit.clear();
            ctx.display.clear();
            ctx.description.clear();
        } else if (t.name == "test") {
            ctx.test = t.attr["name"];
            ctx.unit = t.attr["unit"];
            ctx.display = t.attr["display"];
            ctx.description = t.attr["description"];
        } else if (t.name == "metric") {
            ResultEntry e = ctx;
            e.metric = t.attr["name"];
            e.metricDescription = t.attr["info"];
            if (t.attr.count("status")) {
                e.status = statusFromString(t.attr["status"]);
                e.reason = t.attr["reason"];
            } else {
                e.status = ResultStatus::Ok;
                if (!parseFloatClassic(t.text, e.value))
                    continue;
            }
            if (rowComplete(e))
                store.push_back(e);
        }
    }
    flushDevice();
    warnEmpty(store, filename);
    return store;
}

ResultStore loadResultFile(const std::string &filename, DeviceInfoStore *devices)
{
    auto endsWith = [&](const char *ext) {
        const size_t n = std::strlen(ext);
        if (filename.size() < n)
            return false;
        std::string tail = filename.substr(filename.size() - n);
        for (auto &ch : tail)
            ch = (char)std::tolower((unsigned char)ch);
        return tail == ext;
    };
    if (endsWith(".csv"))
        return loadCsv(filename);
    if (endsWith(".xml"))
        return loadXml(filename, devices);
    return loadJson(filename, devices);
}
